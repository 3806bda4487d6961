#!/usr/bin/env python
"""Benchmark of the MoE-layer decode hot path on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--layers L] [--tokens T]

Workload (N = 1): ragged batched MoE decode — T = 64 concurrent sequences, one token each, through L distinct
MoE layers (512 IQ2_XXS experts, top-10, Q6_K shared expert) whose router logits are DRAWN so that per-expert token
counts follow Zipf(1.1). One step = one pass of the batch through all L layers; the L layers' weights (L x 415 MB) are
far larger than L2, so every step reads its experts from HBM. Prints ONE JSON line.

Other workloads (--workload): moe_b1 (one token through the same layers, router computed), deltanet (gated DeltaNet
decode step, batch 1 and 8), decode48 (48-layer model, greedy decode at a long context), prefill (chunked prefill of
the same model). N > 1 (torchrun): the default workload under expert parallelism, 64 tokens per rank.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "moe_layer_decode_tokens_per_s"
UNIT = "tokens/s"
HBM_PEAK_FALLBACK = 6650.0


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return HBM_PEAK_FALLBACK, "fallback"


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 200 ms while the timed region runs."""
    Q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            time.sleep(0.25)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], 0, set()
        for r in self.rows:
            try:
                sm.append(int(float(r[0])))
                mx = max(mx, int(float(r[1])))
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[2:6]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            except Exception:
                pass
        return {"sm_mhz": int(statistics.median(sm)) if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons), "samples": len(sm)}


def zipf_unique_experts(logits: np.ndarray, top_k: int) -> int:
    sel = np.argpartition(-logits, top_k - 1, axis=1)[:, :top_k]
    return int(np.unique(sel).size)


def algorithmic_bytes(dims, ntok: int, unique: int, router_computed: bool):
    """Bytes one MoE layer pass must move: distinct selected experts + shared expert + activations in/out (+ router)."""
    from dwarfstar_red_lite_b200.synth import row_bytes
    gu = dims.ffn * row_bytes(dims.type_gu, dims.hidden)
    dn = dims.hidden * row_bytes(dims.type_down, dims.ffn)
    sh = 2 * dims.ffn_sh * row_bytes(dims.type_sh, dims.hidden) + dims.hidden * row_bytes(dims.type_sh, dims.ffn_sh)
    total = unique * (2 * gu + dn) + sh + dims.hidden * 4 + ntok * 2 * dims.hidden * 4
    if router_computed:
        total += dims.n_expert * dims.hidden * 4
    return {"layer": total, "gateup": unique * 2 * gu + ntok * dims.hidden * 4, "down": unique * dn}


def cpu_sample(layer_host, x: np.ndarray, logits: np.ndarray, threads: int, budget_s: float):
    """Oracle port of ffn() (native/redlite_native_engine_cpu.c:329-386) over as many tokens of the batch as fit the budget."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as ol
    view = ol.moe_layer_c(layer_host)
    t0 = time.perf_counter()
    n = 0
    while n < x.shape[0]:
        ol.moe_ffn(layer_host, x[n], threads=threads, logits_in=logits[n], view=view)
        n += 1
        if time.perf_counter() - t0 > budget_s:
            break
    dt = time.perf_counter() - t0
    return n / dt, n, dt


def host_layer_from_device(tensors: dict, dims):
    from dwarfstar_red_lite_b200.synth import MoeLayer
    g = lambda k: tensors[k].cpu().numpy()
    return MoeLayer(dims, g("router"), g("gate").reshape(dims.n_expert, -1), g("up").reshape(dims.n_expert, -1),
                    g("down").reshape(dims.n_expert, -1), g("sh_gate_inp"), g("sh_gate").reshape(dims.ffn_sh, -1),
                    g("sh_up").reshape(dims.ffn_sh, -1), g("sh_down").reshape(dims.hidden, -1))


def run_reference(args):
    """The reference arm: the CPU path of the same workload (oracle port, every host thread), bounded sample per step."""
    from dwarfstar_red_lite_b200 import synth
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    dims = synth.MoeDims()
    threads = os.cpu_count() or 1
    layer = synth.moe_layer(1234, dims)
    rng = np.random.default_rng(1)
    x = rng.normal(0, 1, size=(args.tokens, dims.hidden)).astype(np.float32)
    logits = synth.zipf_routing_logits(77, args.tokens)
    sample = max(1, min(args.tokens, args.ref_tokens))
    for _ in range(args.warmup):
        cpu_sample(layer, x[:1], logits[:1], threads, 1e9)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_sample(layer, x[:sample], logits[:sample], threads, 1e9)
    dt = time.perf_counter() - t0
    value = sample * args.steps / dt
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            # a step of the GPU arm is the whole batch through every layer; the CPU sample is scaled to that step
            "ms_per_step": 1e3 * args.tokens * args.layers / value, "ms_per_sampled_step": 1e3 * dt / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
            "config": workload_config(args, dims),
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                             "sample": f"{sample} of the {args.tokens} tokens of one layer per step (oracle port of ffn(); the reference's own routed CPU path rejects IQ2_XXS experts)"},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def workload_config(args, dims):
    return {"workload": "ragged batched MoE decode (BASELINE configs[1]): %d sequences x 1 token, %d experts top-%d IQ2_XXS + Q6_K shared expert, "
                        "router logits drawn Zipf(1.1)" % (args.tokens, dims.n_expert, dims.top_k),
            "tokens_per_step_per_gpu": args.tokens, "layers_per_step": args.layers, "hidden": dims.hidden, "ffn": dims.ffn,
            "l2_policy": "inputs larger than L2: each step sweeps %d distinct layers' experts" % args.layers,
            "parallelism": "single GPU" if args.gpus == 1 else f"ep{args.gpus}"}


def run_ep(args, world, rank, local):
    """N > 1: expert parallelism, all-gather form. Every rank keeps its own 64 tokens (weak scaling) and 512 / N experts of
    every layer; per layer one all-gather of the token rows and one reduce-scatter of the partial outputs over NCCL, no
    host synchronisation inside a step. Placement: interleaved (expert e on rank e % N, the default) or contiguous
    (expert e on rank e // (512 / N)); --ep-permute draws the routing over a random permutation of the expert ids, so
    that popularity is not ordered by id. Timed with CUDA events per rank, maximum over ranks; before the timed region
    rank 0 checks layer 0's output of its first tokens against the CPU oracle."""
    import torch
    import torch.distributed as dist
    import dwarfstar_red_lite_b200 as rc
    from dwarfstar_red_lite_b200 import ep, redcuda as rcm, synth, synth_device
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    rc.set_codebooks(device=local)
    dims = synth.MoeDims()
    L, T = args.layers, args.tokens
    ec = dims.n_expert // world
    contiguous = args.ep_placement == "contiguous"
    perm = np.random.default_rng(4242).permutation(dims.n_expert) if args.ep_permute else np.arange(dims.n_expert)

    def owner_of(ids):           # rank that holds expert id
        return ids // ec if contiguous else ids % world

    def global_id(r, i):         # id of the i-th expert of rank r's shard
        return r * ec + i if contiguous else r + i * world

    layers = []
    for l in range(L):
        tens = synth_device.moe_layer_tensors(1000 + l, dims, dev, expert_begin=rank * ec, expert_count=ec)
        m = rc.MoeLayer(device_tensors=tens, dims=dims, max_tokens=T * world, expert_begin=rank * ec if contiguous else rank, expert_count=ec,
                        expert_stride=1 if contiguous else world)
        layers.append(m if args.ep_impl == "c" else ep.EpGatherMoeLayer(m, rank, world, T))
        del tens

    def drawn_logits(l, r):
        lg = synth.zipf_routing_logits(500 + l + 1000 * r, T)
        return lg[:, np.argsort(perm)] if args.ep_permute else lg      # column e of the result = popularity rank perm^-1(e)

    logits_h = np.stack([drawn_logits(l, rank) for l in range(L)])
    gx = torch.Generator(device=dev)
    gx.manual_seed(7 + rank)
    x_d = torch.randn(L, T, dims.hidden, device=dev, generator=gx)
    logits_d = torch.from_numpy(np.ascontiguousarray(logits_h)).to(dev)

    if args.ep_impl == "c":          # one C call per step: every launch and both collectives of every layer queued by the library
        ctx = ep.EpStep(layers, rank, world, T, exchange=args.ep_exchange)
        ctx.bind(x_d, logits_d)

        def step(mark=None):
            ctx.step()
    else:

        def step(mark=None):
            for l in range(L):
                layers[l].forward(x_d[l], logits=logits_d[l], mark=mark)

    # ---- parity on the devices: layer 0's output of rank 0's first tokens against the oracle port of ffn()
    parity = None
    out0 = (ctx.layer_forward(0, x_d[0], logits_d[0]) if args.ep_impl == "c" else layers[0].forward(x_d[0], logits=logits_d[0])).clone()
    torch.cuda.synchronize()
    dist.barrier()
    if rank == 0 and not args.no_cpu:
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        import oracle_lib as ol
        from dwarfstar_red_lite_b200.synth import MoeLayer
        full = {}
        for r in range(world):       # every rank's shard of layer 0, regenerated from its seed, placed at its experts' global ids
            tens = synth_device.moe_layer_tensors(1000, dims, dev, expert_begin=r * ec, expert_count=ec)
            for k in ("gate", "up", "down"):
                a = tens[k].cpu().numpy().reshape(ec, -1)
                if k not in full:
                    full[k] = np.empty((dims.n_expert, a.shape[1]), np.uint8)
                for i in range(ec):
                    full[k][global_id(r, i)] = a[i]
            if r == 0:
                rest = {k: tens[k].cpu().numpy() for k in ("router", "sh_gate_inp", "sh_gate", "sh_up", "sh_down")}
            del tens
        host = MoeLayer(dims, rest["router"], full["gate"], full["up"], full["down"], rest["sh_gate_inp"], rest["sh_gate"].reshape(dims.ffn_sh, -1),
                        rest["sh_up"].reshape(dims.ffn_sh, -1), rest["sh_down"].reshape(dims.hidden, -1))
        view = ol.moe_layer_c(host)
        ntest, worst, ids_ok = min(4, T), 0.0, True
        x0, got = x_d[0].cpu().numpy(), out0.cpu().numpy()
        for t in range(ntest):
            ro, rid, _, _ = ol.moe_ffn(host, x0[t], threads=os.cpu_count() or 1, logits_in=logits_h[0][t], view=view)
            worst = max(worst, float(np.max(np.abs(got[t] - ro)) / np.max(np.abs(ro))))
        parity = {"layer": 0, "tokens_checked": ntest, "max_rel_err_vs_cpu_oracle": worst, "bound": 1e-3, "ok": bool(worst <= 1e-3)}
        del full, host

    n0 = rcm.lib().redcuda_launch_count()
    step()
    launches_per_step = rcm.lib().redcuda_launch_count() - n0
    for _ in range(args.warmup - 1):
        step()
    torch.cuda.synchronize()
    dist.barrier()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        step()
        side.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(local) as clocks:
            torch.cuda.synchronize()
            t_host0 = time.perf_counter()
            e0.record(side)
            for _ in range(args.steps):
                step()
            e1.record(side)
            t_enqueue = (time.perf_counter() - t_host0) / args.steps        # host time to queue a step (no synchronisation inside)
            torch.cuda.synchronize()
        # ---- phase shares of one more step (events at the phase boundaries on this stream; outside the timed region)
        marks = []

        def mark(name):
            ev = torch.cuda.Event(enable_timing=True)
            ev.record(side)
            marks.append((name, ev))

        phases = {}
        if args.ep_impl == "c":       # per-kernel CUDA events of the library around one more step (collectives included)
            rcm.profile_enable(True)
            step()
            side.synchronize()
            for name, (_, ms_k) in rcm.profile_report().items():
                phases[name] = ms_k
            rcm.profile_enable(False)
        else:
            mark("begin")
            step(mark)
            side.synchronize()
    for (_, a), (name, bb) in zip(marks[:-1], marks[1:]):
        phases[name] = phases.get(name, 0.0) + a.elapsed_time(bb)
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    # pairs this rank's experts served per layer (from the drawn logits of every rank: the same seeds on every rank)
    mine = 0
    for r in range(world):
        for l in range(L):
            lg = logits_h[l] if r == rank else drawn_logits(l, r)
            top = np.argpartition(-lg, dims.top_k - 1, axis=1)[:, :dims.top_k]
            mine += int(np.sum(owner_of(top) == rank))
    pairs = torch.tensor([mine / L], device=dev)
    enq = torch.tensor([t_enqueue * 1e3], device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    dist.all_reduce(enq, op=dist.ReduceOp.MAX)
    allpairs = [torch.zeros_like(pairs) for _ in range(world)]
    dist.all_gather(allpairs, pairs)
    dist.barrier()
    if rank == 0:
        ms_per_step = float(ms.item()) / args.steps
        value = T * world * L / (ms_per_step * 1e-3)
        tot = sum(phases.values()) or 1.0
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": dict(workload_config(args, dims), experts_per_gpu=ec,
                               expert_placement="contiguous (expert e on rank e // (512 / N))" if contiguous else "interleaved (expert e on rank e % N)",
                               routing_ids_permuted=bool(args.ep_permute),
                               pairs_served_per_rank_per_layer=[float(p.item()) for p in allpairs], cuda_graph=False,
                               step_driver="one C call per step (redcuda_ep_step)" if args.ep_impl == "c" else "Python loop over torch.distributed calls",
                               exchange_kind=(ctx.exchange if args.ep_impl == "c" else "nccl"),
                               exchange="per layer: all-gather of the token rows (int8 digits + scales, router ids / weights), reduce-scatter of the partial outputs; "
                                        "peer = stores into the other ranks' memory over NVLink with flag words inside the compute kernels, nccl = ncclAllGather / ncclReduceScatter; no host synchronisation"),
                "roofline": None, "cpu_baseline": None, "parity": parity,
                "breakdown": {"host_enqueue_ms_per_step_max_over_ranks": float(enq.item()), "device_ms_per_step": ms_per_step,
                              "rank0_phase_ms_per_step": {k: round(v, 3) for k, v in phases.items()},
                              "rank0_phase_share": {k: round(v / tot, 3) for k, v in phases.items()}},
                "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                        "note": "multi-GPU runs keep activations on the devices; the host-buffer path is measured at N=1"},
                "gpu_launches": int(launches_per_step * args.steps), "clocks": clocks.summary()}
        print(json.dumps(line), flush=True)
    if args.ep_impl == "c":
        ctx.close()
    dist.destroy_process_group()


def run_decode48(args):
    """BASELINE configs[3]: the whole 48-layer random-init model, batch 1, greedy decode at a long context. The model is
    written as a synthetic GGUF file (seeded), opened through rl_engine_open, and decoded with
    rl_engine_generate_greedy; the CPU baseline is the oracle port of rl_engine_cpu_step on the same file."""
    import dwarfstar_red_lite_b200 as rc
    from dwarfstar_red_lite_b200 import gguf_writer, synth
    from dwarfstar_red_lite_b200.engine import Engine
    os.environ.setdefault("RL_KV_F16", "1")
    dims = synth.ModelDims(n_layer=args.layers, context=args.context)
    tmp = os.environ.get("REDCUDA_TMP", "/tmp")
    path = os.path.join(tmp, f"redcuda_synth_{args.layers}l_seed{args.seed}.gguf")
    t0 = time.perf_counter()
    if not os.path.exists(path):
        size = gguf_writer.write_gguf_streaming(path, args.seed, dims)
    else:
        size = os.path.getsize(path)
    t_write = time.perf_counter() - t0
    rc.set_codebooks()
    t0 = time.perf_counter()
    eng = Engine(path, context=dims.context)
    t_open = time.perf_counter() - t0
    info = eng.info
    new_tokens, start_pos = args.new_tokens, max(0, dims.context - args.new_tokens - 1)
    result = {}
    # ---- parity: greedy tokens from an empty state against the CPU oracle
    check = None
    if args.check_steps > 0:
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        import oracle_lib as ol
        om = ol.OracleModel(gguf_writer.load_gguf(path, dims), kv_f16=True, context=dims.context)
        got, _ = eng.generate_greedy(args.first_token, args.check_steps)        # free-running greedy decode on the GPU
        eng.reset()
        # teacher-forced replay: both sides are fed the oracle's tokens, so one near-tie cannot hide what follows
        tok, want, agree, ties, worst_layer, worst_logit, id_mismatch, t0 = args.first_token, [], 0, [], 0.0, 0.0, 0, time.perf_counter()
        # Every router mismatch with the margin by which the ORACLE's own logits prefer its choice (the smallest gap between an
        # expert only the oracle selected and one only the GPU selected; for a pure order swap the gap of the swapped pair) and
        # the layer-output error just upstream. Both sides keep their own K/V and DeltaNet states, so everything after the
        # first mismatch also carries the flipped expert's contribution: `clean_noise` is the error measured before it.
        margins, first_mismatch, clean_noise = [], None, 0.0
        for i in range(args.check_steps):
            gl = eng.step(tok)
            ml = om.step(tok, threads=os.cpu_count() or 1)
            upstream = 0.0
            for l in range(info.n_layer):
                a_, b_ = eng.layer_out(l), om.layer_out(l)
                gi, ci = eng.router_ids(l), om.router_ids(l)
                if not np.array_equal(gi, ci):
                    id_mismatch += 1
                    lg = om.router_logits(l)
                    only_c, only_g = [e_ for e_ in ci if e_ not in gi], [e_ for e_ in gi if e_ not in ci]
                    if only_c:
                        margin = float(min(lg[e_] for e_ in only_c) - max(lg[e_] for e_ in only_g))
                    else:
                        swapped = [k_ for k_ in range(len(ci)) if gi[k_] != ci[k_]]
                        margin = float(max(abs(lg[ci[k_]] - lg[gi[k_]]) for k_ in swapped))
                    rec = {"step": i, "layer": l, "margin": margin, "same_experts": not only_c, "upstream_rel_err": upstream}
                    margins.append(rec)
                    if first_mismatch is None:
                        first_mismatch = rec
                err_l = float(np.max(np.abs(a_ - b_)) / np.max(np.abs(b_)))
                if first_mismatch is None:
                    clean_noise = max(clean_noise, err_l)
                upstream = err_l
                worst_layer = max(worst_layer, err_l)
            worst_logit = max(worst_logit, float(np.max(np.abs(gl - ml))))
            top2 = np.partition(ml, -2)[-2:]
            if int(np.argmax(gl)) == int(np.argmax(ml)):
                agree += 1
            else:
                ties.append({"step": i, "top2_gap": float(top2[1] - top2[0])})
            tok = int(np.argmax(ml))
            want.append(tok)
        cpu_s = (time.perf_counter() - t0) / args.check_steps
        same = int(np.sum(np.array(want) == got))
        first_diff = next((i for i, (a_, b_) in enumerate(zip(want, got)) if a_ != b_), None)
        check = {"greedy_steps": args.check_steps, "free_running_tokens_equal": same, "first_difference": first_diff,
                 "teacher_forced_argmax_equal": agree, "argmax_differences": ties, "max_layer_rel_err": worst_layer, "max_logit_abs_err": worst_logit,
                 "router_id_layer_mismatches": id_mismatch, "router_selections_checked": args.check_steps * int(info.n_layer),
                 "first_router_mismatch": first_mismatch, "max_layer_rel_err_before_first_mismatch": clean_noise,
                 "mismatch_margins": {"count": len(margins), "max": max((m_["margin"] for m_ in margins), default=None),
                                      "median": float(np.median([m_["margin"] for m_ in margins])) if margins else None,
                                      "same_experts_other_order": int(sum(m_["same_experts"] for m_ in margins)),
                                      "first_20": margins[:20]},
                 "s_per_token_both_sides": cpu_s}
        eng.reset()
        del om
    # ---- timed decode at long context
    rng = np.random.default_rng(args.seed)
    for _ in range(args.warmup):
        eng.set_position(start_pos)
        eng.generate_greedy(int(rng.integers(dims.vocab)), 4)
    times = []
    with ClockSampler(0) as clocks:
        for _ in range(args.steps):
            eng.set_position(start_pos)
            _, ms = eng.generate_greedy(int(rng.integers(dims.vocab)), new_tokens)
            times.append(ms)
    ms_run = float(np.median(times))
    tok_s = new_tokens / (ms_run * 1e-3)
    eng.set_position(dims.context - 1 - new_tokens // 2)
    step_bytes = eng.step_bytes()
    # ---- end to end per token: rl_engine_step with the logits copied to the host every token
    eng.set_position(start_pos)
    logits = np.empty(info.vocab, np.float32)
    tok, t0, n_e2e = 5, time.perf_counter(), min(32, new_tokens)
    for _ in range(n_e2e):
        eng.step(tok, logits=logits)
        tok = int(np.argmax(logits))
    e2e_tok_s = n_e2e / (time.perf_counter() - t0)
    # ---- CPU baseline: the oracle port, all host threads, a bounded number of tokens from an empty state
    cpu = None
    if not args.no_cpu:
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        import oracle_lib as ol
        om = ol.OracleModel(gguf_writer.load_gguf(path, dims), kv_f16=True, context=dims.context)
        threads = os.cpu_count() or 1
        t0, n = time.perf_counter(), 0
        tok = 5
        while n < 8 and (n == 0 or time.perf_counter() - t0 < args.cpu_budget_s):
            tok = int(np.argmax(om.step(tok, threads=threads)))
            n += 1
        dt = time.perf_counter() - t0
        cpu = {"value": n / dt, "unit": "tokens/s", "cores": threads, "kind": "port",
               "sample": f"{n} greedy tokens from an empty state in {dt:.1f} s (oracle port of rl_engine_cpu_step; short context, which favours the CPU)"}
    peak, peak_kind = measured_peak()
    gbs = step_bytes * tok_s / 1e9
    line = {"metric": "decode_tokens_per_s", "value": tok_s, "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_run, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"BASELINE configs[3]: {info.n_layer}-layer Qwen3-Next-shaped random-init model, batch 1, greedy, {new_tokens} new tokens ending at context {dims.context}, fp16 KV",
                       "gguf_bytes": size, "write_s": round(t_write, 1), "open_s": round(t_open, 1), "l2_policy": "one token reads ~%.2f GB of weights and state" % (step_bytes / 1e9)},
            "roofline": {"bound": "hbm", "kernel": "whole decode step", "achieved": gbs, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": gbs / peak,
                         "traffic": None, "bytes_per_token": step_bytes},
            "cpu_baseline": cpu, "e2e": {"value": e2e_tok_s, "unit": "tokens/s", "h2d_bytes_per_step": 4, "d2h_bytes_per_step": int(info.vocab * 4 + info.n_layer * info.hidden * 4)},
            "parity": check, "gpu_launches": None, "clocks": clocks.summary()}
    print(json.dumps(line), flush=True)
    eng.close()


def run_prefill(args):
    """BASELINE configs[4] on one GPU: chunked prefill of a random prompt through the 48-layer random-init model
    (rl_engine_prefill; chunk = --prefill-batch tokens). Tokens/s over the whole prompt, the last token's logits copied
    to the host. The CPU baseline is the oracle port stepping a few prompt tokens (the reference's CPU prefill is
    token by token as well)."""
    import dwarfstar_red_lite_b200 as rc
    from dwarfstar_red_lite_b200 import gguf_writer, synth
    from dwarfstar_red_lite_b200.engine import Engine
    os.environ.setdefault("RL_KV_F16", "1")
    n_prompt = args.prompt_tokens
    dims = synth.ModelDims(n_layer=args.layers, context=max(args.context, n_prompt + 8))
    tmp = os.environ.get("REDCUDA_TMP", "/tmp")
    path = os.path.join(tmp, f"redcuda_synth_{args.layers}l_seed{args.seed}.gguf")
    t0 = time.perf_counter()
    size = os.path.getsize(path) if os.path.exists(path) else gguf_writer.write_gguf_streaming(path, args.seed, dims)
    t_write = time.perf_counter() - t0
    rc.set_codebooks()
    eng = Engine(path, context=dims.context, prefill_batch=args.prefill_batch)
    info, chunk = eng.info, eng.prefill_batch
    rng = np.random.default_rng(args.seed)
    prompt = rng.integers(0, dims.vocab, n_prompt).astype(np.uint32)
    check = None
    if args.check_steps > 0:
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        import oracle_lib as ol
        om = ol.OracleModel(gguf_writer.load_gguf(path, dims), kv_f16=True, context=dims.context)
        n = args.check_steps
        gl = eng.prefill(prompt[:n])
        for t in prompt[:n]:
            ml = om.step(int(t), threads=os.cpu_count() or 1)
        worst = max(float(np.max(np.abs(eng.layer_out(l) - om.layer_out(l))) / np.max(np.abs(om.layer_out(l)))) for l in range(info.n_layer))
        ids = sum(int(not np.array_equal(eng.router_ids(l), om.router_ids(l))) for l in range(info.n_layer))
        # the first layer whose selection differs, with the margin by which the oracle's own logits prefer its choice and the
        # error of the layers before it (what follows a flipped expert is no longer rounding noise)
        first, clean = None, 0.0
        for l in range(info.n_layer):
            gi, ci = eng.router_ids(l), om.router_ids(l)
            if not np.array_equal(gi, ci):
                lg = om.router_logits(l)
                only_c, only_g = [e_ for e_ in ci if e_ not in gi], [e_ for e_ in gi if e_ not in ci]
                margin = float(min(lg[e_] for e_ in only_c) - max(lg[e_] for e_ in only_g)) if only_c else \
                    float(max(abs(lg[ci[k_]] - lg[gi[k_]]) for k_ in range(len(ci)) if gi[k_] != ci[k_]))
                first = {"layer": l, "margin": margin, "same_experts": not only_c}
                break
            clean = max(clean, float(np.max(np.abs(eng.layer_out(l) - om.layer_out(l))) / np.max(np.abs(om.layer_out(l)))))
        check = {"prompt_tokens": n, "chunk": chunk, "max_layer_rel_err_last_token": worst, "max_logit_abs_err": float(np.max(np.abs(gl - ml))),
                 "argmax_equal": bool(int(np.argmax(gl)) == int(np.argmax(ml))), "router_id_layer_mismatches_last_token": ids,
                 "first_router_mismatch": first, "max_layer_rel_err_before_first_mismatch": clean}
        del om
    for _ in range(args.warmup):
        eng.reset()
        eng.prefill(prompt[: min(n_prompt, 2 * chunk)])
    times = []
    launches0 = rc.lib().redcuda_launch_count()
    with ClockSampler(0) as clocks:
        for _ in range(args.steps):
            eng.reset()
            t0 = time.perf_counter()
            eng.prefill(prompt)
            times.append((time.perf_counter() - t0) * 1e3)
    launches = (rc.lib().redcuda_launch_count() - launches0) // max(1, args.steps)
    ms_run = float(np.median(times))
    tok_s = n_prompt / (ms_run * 1e-3)
    cpu = None
    if not args.no_cpu:
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        import oracle_lib as ol
        om = ol.OracleModel(gguf_writer.load_gguf(path, dims), kv_f16=True, context=dims.context)
        threads = os.cpu_count() or 1
        t0, n = time.perf_counter(), 0
        while n < 8 and (n == 0 or time.perf_counter() - t0 < args.cpu_budget_s):
            om.step(int(prompt[n]), threads=threads)
            n += 1
        dt = time.perf_counter() - t0
        cpu = {"value": n / dt, "unit": "tokens/s", "cores": threads, "kind": "port",
               "sample": f"the first {n} prompt tokens in {dt:.1f} s (oracle port of rl_engine_cpu_step, token by token; short context, which favours the CPU)"}
    # weight bytes one chunk has to read: every dense matrix once, plus the experts the chunk's tokens select (expected count
    # under uniform routing); states and K/V are small beside them
    n_chunks = (n_prompt + chunk - 1) // chunk
    per_expert = eng.full_residency_mib() * (1 << 20) / (info.n_layer * info.n_expert)
    uniq = info.n_expert * (1.0 - (1.0 - info.top_k / info.n_expert) ** chunk)
    eng.set_position(0)
    dense_bytes = eng.step_bytes() - per_expert * info.top_k * info.n_layer
    chunk_bytes = dense_bytes + per_expert * uniq * info.n_layer
    peak, peak_kind = measured_peak()
    gbs = chunk_bytes * n_chunks / (ms_run * 1e-3) / 1e9
    line = {"metric": "prefill_tokens_per_s", "value": tok_s, "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_run, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"BASELINE configs[4] on one GPU: chunked prefill of {n_prompt} random tokens, chunks of {chunk}, {info.n_layer}-layer Qwen3-Next-shaped random-init model, fp16 KV",
                       "gguf_bytes": size, "write_s": round(t_write, 1), "l2_policy": "one chunk reads ~%.2f GB of weights" % (chunk_bytes / 1e9)},
            "roofline": {"bound": "hbm", "kernel": "whole prefill (weight bytes per chunk x chunks)", "achieved": gbs, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                         "frac": gbs / peak, "traffic": None, "bytes_per_chunk": chunk_bytes},
            "cpu_baseline": cpu, "e2e": {"value": tok_s, "unit": "tokens/s", "h2d_bytes_per_step": int(n_prompt * 8), "d2h_bytes_per_step": int(info.vocab * 4 + (2 * info.n_layer + 2) * info.hidden * 4),
                                         "note": "the timed call is the host API itself: prompt ids from host memory, logits and mirrors back"},
            "parity": check, "gpu_launches": int(launches), "clocks": clocks.summary()}
    print(json.dumps(line), flush=True)
    eng.close()


def run_prefill_ep(args, world, rank, local):
    """BASELINE configs[4] under expert parallelism: every rank prefills its OWN prompt through its own engine, which holds
    the dense weights and a contiguous share of every layer's experts; per layer the chunk's token rows of all ranks are
    exchanged (all-gather form, see run_ep). Weak scaling: N prompts of --prompt-tokens tokens. Timed per rank around the
    whole prefill call, maximum over ranks. Rank 0 checks the first tokens against the CPU oracle."""
    import torch
    import torch.distributed as dist
    import dwarfstar_red_lite_b200 as rc
    from dwarfstar_red_lite_b200 import ep, gguf_writer, synth
    from dwarfstar_red_lite_b200.engine import Engine
    os.environ.setdefault("RL_KV_F16", "1")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    n_prompt = args.prompt_tokens
    dims = synth.ModelDims(n_layer=args.layers, context=max(args.context, n_prompt + 8))
    tmp = os.environ.get("REDCUDA_TMP", "/tmp")
    path = os.path.join(tmp, f"redcuda_synth_{args.layers}l_seed{args.seed}.gguf")
    if rank == 0 and not os.path.exists(path):
        gguf_writer.write_gguf_streaming(path, args.seed, dims)
    dist.barrier()
    rc.set_codebooks(device=local)
    eng = Engine(path, context=dims.context, prefill_batch=args.prefill_batch, ep_rank=rank, ep_world=world)
    info, chunk = eng.info, eng.prefill_batch
    ctx = ep.EpContext(rank, world, chunk, int(info.hidden), int(info.top_k), exchange=args.ep_exchange)
    eng.attach_ep(ctx)
    prompt = np.random.default_rng(args.seed + 100 * rank).integers(0, dims.vocab, n_prompt).astype(np.uint32)
    check = None
    if args.check_steps > 0:          # every rank runs the same call sequence; rank 0 compares with the oracle
        n = args.check_steps
        gl = eng.prefill(prompt[:n])
        if rank == 0:
            sys.path.insert(0, os.path.join(ROOT, "tests"))
            import oracle_lib as ol
            om = ol.OracleModel(gguf_writer.load_gguf(path, dims), kv_f16=True, context=dims.context)
            for t in prompt[:n]:
                ml = om.step(int(t), threads=os.cpu_count() or 1)
            first, clean = None, 0.0
            for l in range(info.n_layer):
                err_l = float(np.max(np.abs(eng.layer_out(l) - om.layer_out(l))) / np.max(np.abs(om.layer_out(l))))
                if not np.array_equal(eng.router_ids(l), om.router_ids(l)):
                    first = l
                    break
                clean = max(clean, err_l)
            check = {"prompt_tokens": n, "first_router_mismatch_layer": first, "max_layer_rel_err_before_first_mismatch": clean,
                     "argmax_equal": bool(int(np.argmax(gl)) == int(np.argmax(ml))), "bound": 1e-3, "ok": bool(clean <= 1e-3)}
            del om
        dist.barrier()
    for _ in range(args.warmup):
        eng.reset()
        eng.prefill(prompt[: min(n_prompt, 2 * chunk)])
    times = []
    launches0 = rc.lib().redcuda_launch_count()
    with ClockSampler(local) as clocks:
        for _ in range(args.steps):
            eng.reset()
            torch.cuda.synchronize()
            dist.barrier()
            t0 = time.perf_counter()
            eng.prefill(prompt)
            times.append((time.perf_counter() - t0) * 1e3)
    launches = (rc.lib().redcuda_launch_count() - launches0) // max(1, args.steps)
    ms = torch.tensor([float(np.median(times))], device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    if rank == 0:
        ms_run = float(ms.item())
        tok_s = n_prompt * world / (ms_run * 1e-3)
        line = {"metric": "prefill_tokens_per_s", "value": tok_s, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms_run, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": f"BASELINE configs[4] under expert parallelism: {world} prompts of {n_prompt} random tokens (one per rank), chunks of {chunk}, "
                                       f"{info.n_layer}-layer Qwen3-Next-shaped random-init model, fp16 KV, experts sharded contiguously ({info.n_expert // world} per rank)",
                           "exchange_kind": ctx.exchange, "l2_policy": "weights far larger than L2"},
                "roofline": None, "cpu_baseline": None, "parity": check,
                "e2e": {"value": tok_s, "unit": "tokens/s", "h2d_bytes_per_step": int(n_prompt * 8), "d2h_bytes_per_step": int(info.vocab * 4 + (2 * info.n_layer + 2) * info.hidden * 4),
                        "note": "the timed call is the host API itself on every rank: prompt ids from host memory, logits and mirrors back"},
                "gpu_launches": int(launches), "clocks": clocks.summary()}
        print(json.dumps(line), flush=True)
    eng.close()
    ctx.close()
    dist.destroy_process_group()


def _timed_graph(torch, step_fn, steps, warmup, device_index):
    """warm up, capture step_fn(stream) into a CUDA graph on a side stream, time `steps` replays with CUDA events"""
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for _ in range(max(1, warmup)):
            step_fn(side.cuda_stream)
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            step_fn(side.cuda_stream)
        graph.replay()
        side.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(device_index) as clocks:
            torch.cuda.synchronize()
            e0.record(side)
            for _ in range(steps):
                graph.replay()
            e1.record(side)
            torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps, clocks.summary()


def measure_config0(torch, layers, dims, x1_d, out1_d, steps, warmup, device_index):
    """One token through every resident layer, router computed (the single-token path: three launches per layer).
    Returns per-layer time, achieved GB/s on the algorithmic bytes of a token-layer and the launches per layer."""
    import dwarfstar_red_lite_b200 as rc
    L, row = len(layers), dims.hidden * 4

    def step(stream):
        for l in range(L):
            layers[l].forward_device(1, x1_d.data_ptr() + l * row, out1_d.data_ptr() + l * row, stream)

    n0 = rc.lib().redcuda_launch_count()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        step(side.cuda_stream)
        side.synchronize()
    launches = (rc.lib().redcuda_launch_count() - n0) / L
    ms, clocks = _timed_graph(torch, step, steps, warmup, device_index)
    us = 1e3 * ms / L
    bytes_layer = algorithmic_bytes(dims, 1, dims.top_k, True)["layer"]
    peak, kind = measured_peak()
    gbs = bytes_layer / (us * 1e-6) / 1e9
    return {"us_per_layer": us, "GBps": gbs, "frac": gbs / peak, "frac_of_nominal_8000": gbs / 8000.0, "launches_per_layer": launches,
            "bytes_per_token_layer": bytes_layer, "layers_per_step": L, "token_layers_per_s": 1e6 / us}, clocks


def measure_deltanet(torch, steps, warmup, device_index):
    """Gated DeltaNet decode step for batch 1 and 8 over enough distinct layer states to exceed L2 (device pointers,
    the allocation-free entry point). Returns {batchB: {...}}, bytes per sequence-layer and the parameter dict."""
    import ctypes as C
    import dwarfstar_red_lite_b200 as rc
    from dwarfstar_red_lite_b200.redcuda import DeltanetParams, f32p
    dev = torch.device("cuda", device_index)
    lib = rc.lib()
    S, groups, rank, d_conv = 128, 16, 32, 4
    d_inner, channels = rank * S, 2 * S * groups + rank * S
    g = torch.Generator(device=dev)
    g.manual_seed(3)
    pd = {"conv_kernel": torch.randn(channels, d_conv, device=dev, generator=g) * 0.5, "dt_bias": torch.zeros(rank, device=dev),
          "ssm_a": -torch.ones(rank, device=dev), "ssm_norm": 1 + 0.1 * torch.randn(S, device=dev, generator=g)}
    P = DeltanetParams(d_conv, S, groups, rank, d_inner, channels, 1e-6, *[C.cast(pd[k].data_ptr(), f32p) for k in ("conv_kernel", "dt_bias", "ssm_a", "ssm_norm")])
    per_seq_bytes = 2 * rank * S * S * 4 + 2 * channels * (d_conv - 1) * 4 + channels * d_conv * 4 + (channels + 2 * d_inner + 2 * rank) * 4
    results, clocks = {}, None
    for B in (1, 8):
        NL = max(8, int(400e6 // (B * rank * S * S * 4)))          # distinct states per step: ~400 MB of state
        qkv = torch.randn(NL, B, channels, device=dev, generator=g)
        z = torch.randn(NL, B, d_inner, device=dev, generator=g)
        ba = torch.randn(NL, B, 2 * rank, device=dev, generator=g)
        conv = torch.randn(NL, B, channels, d_conv - 1, device=dev, generator=g)
        rec = torch.randn(NL, B, rank, S, S, device=dev, generator=g) * 0.05
        out = torch.empty(NL, B, d_inner, device=dev)

        def step(stream):
            for l in range(NL):
                ok = lib.redcuda_deltanet_step_noalloc(C.byref(P), B, qkv[l].data_ptr(), z[l].data_ptr(), ba[l].data_ptr(), conv[l].data_ptr(), rec[l].data_ptr(),
                                                       out[l].data_ptr(), stream)
                assert ok == 1, lib.redcuda_last_error().decode()

        ms, clocks = _timed_graph(torch, step, steps, warmup, device_index)
        seq_layers_s = NL * B / (ms * 1e-3)
        results[f"batch{B}"] = {"seq_layer_steps_per_s": seq_layers_s, "us_per_layer_call": 1e3 * ms / NL, "GBps": seq_layers_s * per_seq_bytes / 1e9, "layers_per_step": NL}
        del qkv, z, ba, conv, rec, out
    return results, per_seq_bytes, pd, clocks


def run_moe_b1(args):
    """BASELINE configs[0]: one routed-MoE FFN layer, batch 1, router computed. A step sweeps `layers` distinct layers
    (weights from HBM, not L2); value = token-layers per second."""
    import torch
    import dwarfstar_red_lite_b200 as rc
    from dwarfstar_red_lite_b200 import redcuda as rcm, synth, synth_device
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    rc.set_codebooks(device=0)
    dims, L = synth.MoeDims(), args.layers
    layers, layer0_host = [], None
    for l in range(L):
        tens = synth_device.moe_layer_tensors(1000 + l, dims, dev)
        layers.append(rc.MoeLayer(device_tensors=tens, dims=dims, max_tokens=1))
        if l == 0 and not args.no_cpu:
            layer0_host = host_layer_from_device(tens, dims)
        del tens
    g = torch.Generator(device=dev)
    g.manual_seed(7)
    x_d = torch.randn(L, 1, dims.hidden, device=dev, generator=g)
    out_d = torch.empty_like(x_d)
    row = dims.hidden * 4
    c0, clocks = measure_config0(torch, layers, dims, x_d, out_d, args.steps, args.warmup, 0)
    value = c0["token_layers_per_s"]
    # per-kernel durations (CUDA events around every launch, eager, separate from the timed region)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        rcm.profile_enable(True)
        for _ in range(3):
            for l in range(L):
                layers[l].forward_device(1, x_d.data_ptr() + l * row, out_d.data_ptr() + l * row, side.cuda_stream)
        side.synchronize()
        prof = rcm.profile_report()
        rcm.profile_enable(False)
    kernel_us = {k: round(1e3 * v[1] / v[0], 2) for k, v in prof.items()}
    xh, oh = x_d.cpu().numpy(), np.empty((L, 1, dims.hidden), np.float32)
    t0 = time.perf_counter()
    for l in range(L):
        layers[l].forward(xh[l], out=oh[l])
    e2e_v = L / (time.perf_counter() - t0)
    peak, kind = measured_peak()
    cpu = None
    if layer0_host is not None:
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        import oracle_lib as ol
        view, threads = ol.moe_layer_c(layer0_host), os.cpu_count() or 1
        t0, n = time.perf_counter(), 0
        while time.perf_counter() - t0 < args.cpu_budget_s and n < 64:
            ol.moe_ffn(layer0_host, xh[0][0], threads=threads, view=view)
            n += 1
        cpu = {"value": n / (time.perf_counter() - t0), "unit": UNIT, "cores": threads, "kind": "port", "sample": f"{n} passes of one token through layer 0 (oracle port of ffn())"}
    print(json.dumps({"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e-3 * c0["us_per_layer"] * L,
                      "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                      "config": {"workload": "BASELINE configs[0]: single routed-MoE FFN layer, batch 1, router computed, 512 IQ2_XXS experts top-10 + Q6_K shared expert",
                                 "layers_per_step": L, "l2_policy": f"each step sweeps {L} distinct layers' weights"},
                      "roofline": {"bound": "hbm", "kernel": "whole layer (%d launches)" % round(c0["launches_per_layer"]), "kernel_us_per_launch": kernel_us, "achieved": c0["GBps"],
                                   "peak": peak, "peak_kind": kind, "unit": "GB/s", "frac": c0["frac"], "frac_of_nominal_8000": c0["frac_of_nominal_8000"], "traffic": None,
                                   "bytes_per_token_layer": c0["bytes_per_token_layer"], "us_per_layer": c0["us_per_layer"]},
                      "cpu_baseline": cpu, "e2e": {"value": e2e_v, "unit": UNIT, "h2d_bytes_per_step": L * row, "d2h_bytes_per_step": L * row},
                      "gpu_launches": int(round(c0["launches_per_layer"] * L * args.steps)), "clocks": clocks}), flush=True)


def run_deltanet(args):
    """BASELINE configs[2]: gated DeltaNet decode step (conv + SiLU + L2 norm, delta rule on the 128x128 fp32 states of
    32 value heads, gated RMSNorm) for batch 1 and 8; a step sweeps enough distinct layer states to exceed L2."""
    import torch
    torch.cuda.set_device(0)
    import dwarfstar_red_lite_b200 as rc
    rc.lib()
    results, per_seq_bytes, pd, clocks = measure_deltanet(torch, args.steps, args.warmup, 0)
    S, groups, rank, d_conv = 128, 16, 32, 4
    d_inner, channels = rank * S, 2 * S * groups + rank * S
    cpu = None
    if not args.no_cpu:
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        import oracle_lib as ol
        rng = np.random.default_rng(1)
        p = dict(d_conv=d_conv, d_state=S, n_group=groups, dt_rank=rank, d_inner=d_inner, channels=channels, rms_eps=1e-6,
                 conv_kernel=pd["conv_kernel"].cpu().numpy(), dt_bias=np.zeros(rank, np.float32), ssm_a=-np.ones(rank, np.float32), ssm_norm=pd["ssm_norm"].cpu().numpy())
        cs, rs = rng.normal(0, 1, (channels, d_conv - 1)).astype(np.float32), rng.normal(0, 0.05, (rank, S, S)).astype(np.float32)
        q1, z1, b1 = rng.normal(0, 1, channels).astype(np.float32), rng.normal(0, 1, d_inner).astype(np.float32), rng.normal(0, 1, 2 * rank).astype(np.float32)
        t0, n = time.perf_counter(), 0
        while time.perf_counter() - t0 < min(args.cpu_budget_s, 10.0):
            ol.deltanet_mid(p, q1, z1, b1, cs, rs)
            n += 1
        cpu = {"value": n / (time.perf_counter() - t0), "unit": "sequence-layer steps/s", "cores": 1, "kind": "port", "sample": f"{n} single-sequence steps (oracle port of the deltanet_branch mid-section, one thread as in the reference)"}
    peak, kind = measured_peak()
    b8 = results["batch8"]
    print(json.dumps({"metric": "deltanet_seq_layer_steps_per_s", "value": b8["seq_layer_steps_per_s"], "unit": "sequence-layer steps/s", "n_gpus": 1, "steps": args.steps,
                      "warmup": args.warmup, "ms_per_step": None, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                      "config": {"workload": "BASELINE configs[2]: gated DeltaNet decode step, 16 key / 32 value heads, 128x128 fp32 state per head, batch 1 and 8", "results": results,
                                 "l2_policy": "each step sweeps ~400 MB of distinct states"},
                      "roofline": {"bound": "hbm", "kernel": "DeltaNet decode step", "achieved": b8["GBps"], "peak": peak, "peak_kind": kind, "unit": "GB/s",
                                   "frac": b8["GBps"] / peak, "traffic": None, "bytes_per_sequence_layer": per_seq_bytes, "batch1_GBps": results["batch1"]["GBps"]},
                      "cpu_baseline": cpu, "e2e": None, "gpu_launches": None, "clocks": clocks}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="redcuda", choices=["redcuda", "reference"])
    ap.add_argument("--layers", type=int, default=48)
    ap.add_argument("--tokens", type=int, default=64)
    ap.add_argument("--ref-tokens", type=int, default=8, help="tokens per step of the reference (CPU) arm")
    ap.add_argument("--cpu-budget-s", type=float, default=15.0)
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--workload", default="ragged64", choices=["ragged64", "decode48", "moe_b1", "deltanet", "prefill"],
                    help="ragged64: BASELINE configs[1] (default, the headline); decode48: configs[3], whole-model decode; "
                         "moe_b1: configs[0], one MoE layer at batch 1; deltanet: configs[2]")
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--new-tokens", type=int, default=128)
    ap.add_argument("--check-steps", type=int, default=0, help="decode48: greedy tokens compared with the CPU oracle")
    ap.add_argument("--first-token", type=int, default=7)
    ap.add_argument("--prompt-tokens", type=int, default=8192, help="prefill: prompt length")
    ap.add_argument("--prefill-batch", type=int, default=0, help="prefill: tokens per chunk (0 = engine default)")
    ap.add_argument("--seed", type=int, default=1)
    ap.add_argument("--ep-placement", default="interleaved", choices=["interleaved", "contiguous"], help="N > 1: which rank holds which expert")
    ap.add_argument("--ep-impl", default="c", choices=["c", "python"], help="N > 1: the library's one-call step, or the per-operation Python loop")
    ap.add_argument("--ep-exchange", default="auto", choices=["auto", "peer", "nccl"],
                    help="N > 1, --ep-impl c: exchange through peer memory or through NCCL; auto = peer memory up to 4 ranks, NCCL above "
                         "(measured: 0.85 / 0.80 against 0.75 / 0.72 at 2 / 4 ranks, 0.57 against 0.60 at 8, where waits inside kernels make rank skew cost more)")
    ap.add_argument("--ep-permute", action="store_true", help="N > 1: draw the routing over a random permutation of the expert ids")
    args = ap.parse_args()
    if args.ep_exchange == "auto":
        args.ep_exchange = "peer" if int(os.environ.get("WORLD_SIZE", "1")) <= 4 else "nccl"
    if args.workload == "decode48":
        args.warmup = max(args.warmup, 1)
        return run_decode48(args)
    if args.workload == "prefill":
        world = int(os.environ.get("WORLD_SIZE", "1"))
        if world > 1:
            if args.gpus != world:
                raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
            return run_prefill_ep(args, world, int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")))
        return run_prefill(args)
    if args.workload == "moe_b1":
        return run_moe_b1(args)
    if args.workload == "deltanet":
        return run_deltanet(args)
    args.warmup = max(args.warmup, 3) if args.impl == "redcuda" else args.warmup
    if args.impl == "reference":
        return run_reference(args)

    import torch
    import dwarfstar_red_lite_b200 as rc
    from dwarfstar_red_lite_b200 import redcuda as rcm, synth, synth_device

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if world > 1:
        return run_ep(args, world, rank, local)
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    rc.set_codebooks(device=local)
    dims = synth.MoeDims()
    L, T = args.layers, args.tokens

    # ---- resident layers, inputs, drawn logits
    layers, uniq = [], []
    layer0_host = None
    for l in range(L):
        tens = synth_device.moe_layer_tensors(1000 + l, dims, dev)
        layers.append(rc.MoeLayer(device_tensors=tens, dims=dims, max_tokens=T))
        if l == 0 and not args.no_cpu:
            layer0_host = host_layer_from_device(tens, dims)
        del tens
    torch.cuda.synchronize()
    logits_h = np.stack([synth.zipf_routing_logits(500 + l, T) for l in range(L)])
    uniq = [zipf_unique_experts(logits_h[l], dims.top_k) for l in range(L)]
    gx = torch.Generator(device=dev)
    gx.manual_seed(7)
    x_d = torch.randn(L, T, dims.hidden, device=dev, generator=gx)
    logits_d = torch.from_numpy(logits_h).to(dev)
    out_d = torch.empty(L, T, dims.hidden, device=dev)
    row = T * dims.hidden * 4

    def step(stream):
        for l in range(L):
            layers[l].forward_device(T, x_d.data_ptr() + l * row, out_d.data_ptr() + l * row, stream, logits_ptr=logits_d.data_ptr() + l * T * dims.n_expert * 4)

    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        n0 = rcm.lib().redcuda_launch_count()
        step(side.cuda_stream)
        launches_per_step = rcm.lib().redcuda_launch_count() - n0
        for _ in range(args.warmup - 1):
            step(side.cuda_stream)
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            step(side.cuda_stream)
        graph.replay()
        side.synchronize()
        # ---- timed region: K graph replays, CUDA events on the launching stream
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(local) as clocks:
            torch.cuda.synchronize()
            e0.record(side)
            for _ in range(args.steps):
                graph.replay()
            e1.record(side)
            torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        # ---- per-kernel durations (events around every launch, same stream, same inputs; separate from the timed region)
        rcm.profile_enable(True)
        prof_steps = 3
        for _ in range(prof_steps):
            step(side.cuda_stream)
        side.synchronize()
        prof = rcm.profile_report()
        rcm.profile_enable(False)
    ms_per_step = ms / args.steps
    value = T * L / (ms_per_step * 1e-3)

    # ---- roofline of the dominant kernel (routed gate/up)
    peak, peak_kind = measured_peak()
    ab = [algorithmic_bytes(dims, T, u, False) for u in uniq]
    total_prof_ms = sum(v[1] for v in prof.values()) or 1.0
    shares = {k: round(v[1] / total_prof_ms, 4) for k, v in prof.items()}
    dom = max(prof, key=lambda k: prof[k][1])
    key = {"moe_gateup": "gateup", "moe_down": "down"}.get(dom)
    dom_bytes = float(np.mean([a[key] for a in ab])) if key else float(np.mean([a["layer"] for a in ab]))
    dom_ms = prof[dom][1] / prof[dom][0]
    achieved = dom_bytes / (dom_ms * 1e-3) / 1e9
    layer_bytes = float(np.mean([a["layer"] for a in ab]))
    # The routed experts are held in the nibble layout by default (138 bytes per 256 weights where the GGUF block has
    # 66): `achieved` / `frac` are on the ALGORITHMIC bytes, `bytes_read_per_launch` is what the kernel really reads.
    nib = not os.environ.get("RC_EXPERT_FMT", "nib4").startswith("i")
    real = dom_bytes * (138.0 / 66.0) if (nib and key) else dom_bytes
    # DRAM traffic per launch: ncu (dram__bytes_read + dram__bytes_write) of the nibble-layout kernels on a 2-layer
    # capture: 231.2 MB read + 4.8 MB written by a gate/up launch whose expert records are 230.6 MB, 116.3 + 6.2 MB by a
    # down launch of 115.3 MB; traffic grows with the distinct experts read, so it is scaled by the bytes read.
    ncu_ratio = ({"moe_gateup": 236.0 / 230.6, "moe_down": 122.5 / 115.3} if nib else {"moe_gateup": 114.93 / 105.41, "moe_down": 51.39 / 52.4}).get(dom)
    roofline = {"bound": "hbm", "kernel": dom, "achieved": achieved, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak,
                "frac_of_nominal_8000": achieved / 8000.0, "traffic": real * ncu_ratio if ncu_ratio else None,
                "traffic_source": ("ncu capture of a 2-layer run of the %s kernels, scaled by the bytes read" % ("nibble-layout" if nib else "planar-format")) if ncu_ratio else None,
                "expert_layout": "nib4 (138 B per 256 weights)" if nib else "iq2 (66 B per 256 weights)",
                "bytes_read_per_launch": real, "read_GBps": real / (dom_ms * 1e-3) / 1e9, "read_frac": real / (dom_ms * 1e-3) / 1e9 / peak,
                "bytes_per_launch": dom_bytes, "ms_per_launch": dom_ms,
                "kernel_time_shares": shares,
                "kernel_us_per_layer": {k: round(1e3 * v[1] / (prof_steps * L), 2) for k, v in prof.items()},
                "whole_layer": {"bytes": layer_bytes, "GBps": layer_bytes * L / (ms_per_step * 1e-3) / 1e9,
                                "frac": layer_bytes * L / (ms_per_step * 1e-3) / 1e9 / peak}}

    # ---- end to end through the host API: pinned host buffers in, host buffers out, every layer call synchronous
    xh = torch.randn(L, T, dims.hidden).pin_memory()
    lh = torch.from_numpy(logits_h).pin_memory()
    oh = torch.empty(L, T, dims.hidden).pin_memory()
    xn, ln, on = xh.numpy(), lh.numpy(), oh.numpy()

    def e2e_step():
        for l in range(L):
            layers[l].forward(xn[l], logits_in=ln[l], out=on[l])

    for _ in range(2):
        e2e_step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    e2e_steps = max(3, args.steps // 4)
    for _ in range(e2e_steps):
        e2e_step()
    torch.cuda.synchronize()
    e2e_dt = (time.perf_counter() - t0) / e2e_steps
    e2e = {"value": T * L / e2e_dt, "unit": UNIT, "h2d_bytes_per_step": L * (T * dims.hidden * 4 + T * dims.n_expert * 4),
           "d2h_bytes_per_step": L * T * dims.hidden * 4, "ms_per_step": e2e_dt * 1e3}

    # ---- CPU baseline: the oracle port on this box's host cores, bounded sample of the same workload (layer 0)
    cpu = None
    if layer0_host is not None:
        threads = os.cpu_count() or 1
        v, n, dt = cpu_sample(layer0_host, x_d[0].cpu().numpy(), logits_h[0], threads, args.cpu_budget_s)
        cpu = {"value": v, "unit": UNIT, "cores": threads, "kind": "port",
               "sample": f"{n} of the {T} tokens of layer 0 in {dt:.1f} s (oracle port of ffn(), rows spread over {threads} threads)"}

    # ---- the other single-GPU configurations of the path, measured in the same process on the same resident layers:
    # configs[0] (one token through every layer, router computed; what the >= 70 % target is phrased on) and configs[2]
    # (the DeltaNet decode step). Reported inside `roofline` / `e2e` next to the headline numbers.
    x1_d = torch.randn(L, 1, dims.hidden, device=dev, generator=gx)
    out1_d = torch.empty_like(x1_d)
    c0, _ = measure_config0(torch, layers, dims, x1_d, out1_d, max(5, args.steps // 2), 3, local)
    x1h, o1h = x1_d.cpu().numpy(), np.empty((L, 1, dims.hidden), np.float32)
    for l in range(L):
        layers[l].forward(x1h[l], out=o1h[l])
    t0 = time.perf_counter()
    for l in range(L):
        layers[l].forward(x1h[l], out=o1h[l])
    c0_e2e = L / (time.perf_counter() - t0)
    roofline["config0"] = {k: c0[k] for k in ("us_per_layer", "GBps", "frac", "frac_of_nominal_8000", "launches_per_layer", "bytes_per_token_layer")}
    e2e["config0"] = {"value": c0_e2e, "unit": "token-layers/s", "h2d_bytes_per_step": dims.hidden * 4, "d2h_bytes_per_step": dims.hidden * 4}
    dn, dn_bytes, _, _ = measure_deltanet(torch, max(5, args.steps // 2), 3, local)
    roofline["config2"] = {"batch1": {"us_per_step": dn["batch1"]["us_per_layer_call"], "GBps": dn["batch1"]["GBps"], "frac": dn["batch1"]["GBps"] / peak},
                           "batch8": {"us_per_step": dn["batch8"]["us_per_layer_call"], "GBps": dn["batch8"]["GBps"], "frac": dn["batch8"]["GBps"] / peak},
                           "bytes_per_sequence_layer": dn_bytes}

    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": dict(workload_config(args, dims), unique_experts_per_layer_mean=float(np.mean(uniq))),
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": int(launches_per_step * args.steps),
            "clocks": clocks.summary()}
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
