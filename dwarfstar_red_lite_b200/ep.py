"""Expert parallelism for the ragged-batch MoE layer: one process per GPU, router and shared expert replicated, tokens
stay with their rank. Two forms:

* all-gather form (EpGatherMoeLayer, the one bench.py runs): experts interleaved over the ranks (expert e on rank
  e % world, so a skewed routing loads the ranks evenly); per layer every rank all-gathers the step's token rows with
  their router ids / weights (a decode batch is small: 64 tokens x 8 KB per rank), runs its own experts over the pairs
  that select them, and a reduce-scatter sums the ranks' partial outputs back to the tokens' owners. Two fixed-size
  collectives per layer, nothing data-dependent on the host, so the whole step is queued without a synchronisation.
  EpStep runs the same form through ONE C call per step (redcuda_ep_step: every launch and both collectives of every
  layer queued by the library), which takes the Python / torch.distributed overhead of ~12 operations per layer off the
  host; EpGatherMoeLayer keeps the per-operation Python form for A/B runs and for the CPU (gloo) tests of the data flow.
* dispatch form (EpMoeLayer): experts sharded contiguously (expert e on rank e // (n_expert / world)), pairs sent to
  their experts' ranks by all-to-all with data-dependent split sizes (one host synchronisation per layer).

Per layer: route locally -> (token, expert) pairs sorted by destination rank -> all-to-all of the pair activations and
expert ids (dispatch) -> the shard's expert FFN over the received pairs -> all-to-all of the expert outputs back
(combine) -> per-token weighted sum in router order. This is the multi-GPU form of the reference's single-device pair
layout (expert_start / pair_token / pair_weight, native/redmetal_topk.h:182-190); the reference itself has no
multi-device path. torch.distributed is plumbing only (NCCL on GPUs, gloo in the CPU tests); the compute on either
side of the exchange is the library's (`experts_fn`, `shared_fn`, `combine_fn`).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass
class DispatchPlan:
    order: torch.Tensor          # [P] pair ids (t * top_k + k) sorted by destination rank (stable)
    inverse: torch.Tensor        # [P] position of pair p in the sorted order (row of its result after the combine exchange)
    send_counts: list[int]       # pairs sent to every rank
    recv_counts: list[int]       # pairs received from every rank


def expert_owner(ids: torch.Tensor, n_expert: int, world: int) -> torch.Tensor:
    return (ids.to(torch.int64) // (n_expert // world)).to(torch.int64)


def plan_dispatch(ids: torch.Tensor, n_expert: int, world: int, group=None) -> DispatchPlan:
    """ids [T, top_k] (any integer dtype, on the device that will exchange). One tiny count exchange; the split sizes
    have to be known on the host, so this is the one host synchronisation of a layer."""
    flat = ids.reshape(-1)
    dest = expert_owner(flat, n_expert, world)
    order = torch.argsort(dest, stable=True)
    inverse = torch.empty_like(order)
    inverse[order] = torch.arange(order.numel(), device=order.device, dtype=order.dtype)
    send = torch.bincount(dest, minlength=world).to(torch.int64)
    recv = torch.empty_like(send)
    if world > 1:
        dist.all_to_all_single(recv, send, group=group)
    else:
        recv.copy_(send)
    return DispatchPlan(order, inverse, [int(v) for v in send.tolist()], [int(v) for v in recv.tolist()])


def exchange(rows: torch.Tensor, send_counts: list[int], recv_counts: list[int], group=None) -> torch.Tensor:
    """all-to-all of rows [sum(send_counts), ...] -> [sum(recv_counts), ...]"""
    out = rows.new_empty((sum(recv_counts),) + tuple(rows.shape[1:]))
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=recv_counts, input_split_sizes=send_counts, group=group)
    else:
        out.copy_(rows)
    return out


def ep_moe_forward(x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, n_expert: int, world: int, experts_fn, shared_fn, combine_fn,
                   group=None):
    """x [T, H] float32, ids / weights [T, top_k] from the router.
    experts_fn(pair_x [P, H], pair_expert [P] int32) -> [P, H] unweighted outputs of this rank's experts
    shared_fn(x) -> [T, H] shared-expert part (already gated), or None
    combine_fn(pair_out [P, H], pair_row [P] int32, weights, add) -> [T, H]
    Returns (out [T, H], plan)."""
    T, k = ids.shape
    plan = plan_dispatch(ids, n_expert, world, group)
    tok_of_pair = (plan.order // k)
    send_x = x.index_select(0, tok_of_pair)                                   # activations of the pairs, destination-major
    send_e = ids.reshape(-1).index_select(0, plan.order).to(torch.int32)
    recv_x = exchange(send_x, plan.send_counts, plan.recv_counts, group)
    recv_e = exchange(send_e, plan.send_counts, plan.recv_counts, group)
    shared = shared_fn(x) if shared_fn is not None else None                   # independent of the exchange
    recv_out = experts_fn(recv_x, recv_e) if recv_x.shape[0] else recv_x.new_empty((0, x.shape[1]))
    back = exchange(recv_out, plan.recv_counts, plan.send_counts, group)      # row i = result of pair plan.order[i]
    out = combine_fn(back, plan.inverse.to(torch.int32), weights, shared)
    return out, plan


class EpMoeLayer:
    """One MoE layer under expert parallelism on CUDA: wraps a redcuda MoeLayer that holds this rank's expert shard."""

    def __init__(self, moe_shard, rank: int, world: int, max_tokens: int, group=None):
        self.m, self.rank, self.world, self.group = moe_shard, rank, world, group
        d = moe_shard.dims
        self.dims = d
        dev = torch.device("cuda", torch.cuda.current_device())
        self.ids = torch.empty(max_tokens, d.top_k, dtype=torch.int32, device=dev)
        self.w = torch.empty(max_tokens, d.top_k, dtype=torch.float32, device=dev)
        self.shared = torch.empty(max_tokens, d.hidden, dtype=torch.float32, device=dev)
        self.pair_counts_last = None

    def forward(self, x: torch.Tensor, out: torch.Tensor, logits: torch.Tensor | None = None):
        T = x.shape[0]
        st = torch.cuda.current_stream().cuda_stream
        ids, w = self.ids[:T], self.w[:T]
        self.m.route_device(T, x.data_ptr(), ids.data_ptr(), w.data_ptr(), st, logits_ptr=0 if logits is None else logits.data_ptr())

        def experts_fn(px, pe):
            po = torch.empty_like(px)
            self.m.experts_device(px.shape[0], px.data_ptr(), pe.data_ptr(), po.data_ptr(), st)
            return po

        def shared_fn(xx):
            self.m.shared_device(T, xx.data_ptr(), self.shared.data_ptr(), st)
            return self.shared[:T]

        def combine_fn(back, pair_row, weights, add):
            self.m.combine_device(T, back.data_ptr(), pair_row.data_ptr(), weights.data_ptr(), add.data_ptr(), 0, out.data_ptr(), st)
            return out

        _, plan = ep_moe_forward(x, ids, w, self.dims.n_expert, self.world, experts_fn, shared_fn, combine_fn, self.group)
        self.pair_counts_last = sum(plan.recv_counts)
        return out


def gather_moe_forward(packed: torch.Tensor, hidden: int, top_k: int, world: int, partial_fn, shared_fn, group=None, mark=None):
    """All-gather form of one layer. packed [T, hidden + 2*top_k] float32: the token's activation row followed by its
    router ids (int32 bits) and weights. partial_fn(all_packed [world*T, hidden + 2*top_k]) -> [world*T, hidden] partial
    sums of this rank's experts; shared_fn(packed) -> [T, hidden] or None (runs while the all-gather is in flight).
    mark(name), when given, is called at the phase boundaries (a caller records CUDA events there).
    Returns routed [T, hidden] (+ shared)."""
    T = packed.shape[0]
    if world > 1:
        all_packed = packed.new_empty((world * T, packed.shape[1]))
        work = dist.all_gather_into_tensor(all_packed, packed, group=group, async_op=True)
        shared = shared_fn(packed) if shared_fn is not None else None
        work.wait()
    else:
        all_packed = packed
        shared = shared_fn(packed) if shared_fn is not None else None
    if mark:
        mark("all_gather")
    partial = partial_fn(all_packed)
    if mark:
        mark("experts")
    if world > 1:
        routed = partial.new_empty((T, hidden))
        dist.reduce_scatter_tensor(routed, partial, op=dist.ReduceOp.SUM, group=group)
    else:
        routed = partial
    if mark:
        mark("reduce_scatter")
    return routed if shared is None else routed.add_(shared)


class EpGatherMoeLayer:
    """One MoE layer under the all-gather form on CUDA: wraps a redcuda MoeLayer created with expert_begin = rank,
    expert_stride = world, max_tokens >= world * tokens."""

    def __init__(self, moe_shard, rank: int, world: int, tokens: int, group=None):
        self.m, self.rank, self.world, self.group, self.T = moe_shard, rank, world, group, tokens
        d = moe_shard.dims
        self.dims = d
        dev = torch.device("cuda", torch.cuda.current_device())
        self.width = d.hidden + 2 * d.top_k
        self.packed = torch.zeros(tokens, self.width, dtype=torch.float32, device=dev)       # x | ids | weights
        self.ids = torch.empty(tokens, d.top_k, dtype=torch.int32, device=dev)
        self.w = torch.empty(tokens, d.top_k, dtype=torch.float32, device=dev)
        self.shared = torch.empty(tokens, d.hidden, dtype=torch.float32, device=dev)
        self.partial = torch.empty(world * tokens, d.hidden, dtype=torch.float32, device=dev)
        self.side = torch.cuda.Stream(device=dev)

    def forward(self, x: torch.Tensor, logits: torch.Tensor | None = None, mark=None) -> torch.Tensor:
        """mark(name): optional callback at the phase boundaries route+pack / all_gather / experts / reduce_scatter / add."""
        d, T = self.dims, self.T
        st = torch.cuda.current_stream().cuda_stream
        self.packed[:, :d.hidden].copy_(x)
        self.m.route_device(T, x.data_ptr(), self.ids.data_ptr(), self.w.data_ptr(), st, logits_ptr=0 if logits is None else logits.data_ptr())
        self.packed[:, d.hidden:d.hidden + d.top_k].copy_(self.ids.view(torch.float32))
        self.packed[:, d.hidden + d.top_k:].copy_(self.w)

        def partial_fn(allp):
            n = allp.shape[0]
            base = allp.data_ptr()
            self.m.partial_device(n, base, self.width, base + 4 * d.hidden, base + 4 * (d.hidden + d.top_k), self.width, self.partial.data_ptr(), st)
            return self.partial[:n]

        def shared_fn(pk):
            # the shared expert needs neither the router nor the exchange: it runs on a side stream next to the
            # collectives and the routed experts and is joined before the final add
            self.side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.side):
                self.m.shared_device(T, x.data_ptr(), self.shared.data_ptr(), self.side.cuda_stream)
            return None

        if mark:
            mark("route_pack")
        routed = gather_moe_forward(self.packed, d.hidden, d.top_k, self.world, partial_fn, shared_fn, self.group, mark)
        torch.cuda.current_stream().wait_stream(self.side)
        out = routed.add_(self.shared)
        if mark:
            mark("add")
        return out


class EpContext:
    """The library's exchange context of one rank (redcuda_ep): NCCL communicator, exchange buffers and, for ranks on one
    node, the other ranks' exchange areas mapped through CUDA IPC. The NCCL unique id and the IPC handles travel over
    `group` (any torch.distributed backend). exchange: "peer" = stores into the other ranks' memory over NVLink with flag
    words (2 to 8 ranks), "nccl" = ncclAllGather / ncclReduceScatter."""

    def __init__(self, rank: int, world: int, tokens: int, hidden: int, top_k: int, group=None, exchange: str = "peer"):
        import ctypes as C
        import numpy as np
        from .redcuda import RedcudaError, lib
        self._lib, self._group, self.world, self.rank, self.tokens = lib(), group, world, rank, tokens

        def check(ok):
            if not ok:
                raise RedcudaError(self._lib.redcuda_last_error().decode(errors="replace"))

        dev = torch.device("cuda", torch.cuda.current_device())
        on_dev = world > 1 and dist.get_backend(group) == "nccl"
        uid = torch.zeros(128, dtype=torch.uint8)
        if world > 1:
            if rank == 0:
                buf = (C.c_uint8 * 128)()
                check(self._lib.redcuda_ep_unique_id(buf) == 1)
                uid = torch.from_numpy(np.frombuffer(buf, dtype=np.uint8).copy())
            uid = uid.to(dev) if on_dev else uid
            dist.broadcast(uid, src=0, group=group)
            uid = uid.cpu()
        self.handle = self._lib.redcuda_ep_create(rank, world, uid.numpy().tobytes(), tokens, hidden, top_k)
        check(bool(self.handle))
        self.exchange = "nccl" if world > 1 else "none"
        if world > 1 and exchange == "peer" and world <= 8:
            hb = (C.c_uint8 * 64)()
            check(self._lib.redcuda_ep_ipc_handle(self.handle, hb) == 1)
            mine = torch.from_numpy(np.frombuffer(hb, dtype=np.uint8).copy())
            mine = mine.to(dev) if on_dev else mine
            everyone = torch.empty(world * 64, dtype=torch.uint8, device=mine.device)
            dist.all_gather_into_tensor(everyone, mine, group=group)
            mapped = self._lib.redcuda_ep_attach_peers(self.handle, everyone.cpu().numpy().tobytes()) == 1
            # every rank must use the same exchange: if one could not map the others' areas (IPC not permitted, no peer
            # access), all fall back to NCCL. The all-reduce is also the barrier before the first step.
            agreed = torch.tensor([1 if mapped else 0], dtype=torch.int32, device=dev if on_dev else "cpu")
            dist.all_reduce(agreed, op=dist.ReduceOp.MIN, group=group)
            if int(agreed.item()) == 1:
                self.exchange = "peer"
            elif mapped:
                check(self._lib.redcuda_ep_detach_peers(self.handle) == 1)

    def close(self):
        if self.handle:
            if self.world > 1:
                torch.cuda.synchronize()
                dist.barrier(group=self._group)    # other ranks may still be writing into this rank's exchange area
            self._lib.redcuda_ep_destroy(self.handle)
            self.handle = None


class EpStep:
    """The all-gather form through the library's own step call: one C entry per step queues route, pack, all-gather, the
    shard's experts, reduce-scatter, shared expert and add of every layer. `shards` are redcuda MoeLayer objects created
    with max_tokens >= world * tokens. The NCCL unique id travels from rank 0 over `group` (any backend)."""

    def __init__(self, shards, rank: int, world: int, tokens: int, group=None, exchange: str = "peer"):
        import ctypes as C
        from .redcuda import lib
        self._lib, self._C = lib(), C
        d = shards[0].dims
        self.dims, self.T, self.world, self.shards = d, tokens, world, shards
        self.ctx = EpContext(rank, world, tokens, d.hidden, d.top_k, group, exchange)
        self._h, self.exchange = self.ctx.handle, self.ctx.exchange
        dev = torch.device("cuda", torch.cuda.current_device())
        n = len(shards)
        self._layers = (C.c_void_p * n)(*[m.handle for m in shards])
        self.out = torch.empty(n, tokens, d.hidden, dtype=torch.float32, device=dev)
        self._outs = (C.c_void_p * n)(*[self.out[l].data_ptr() for l in range(n)])

    def bind(self, x: torch.Tensor, logits: torch.Tensor | None = None):
        """x [layers][tokens][hidden] (every layer its own input, as the benchmark feeds them), logits [layers][tokens][n_expert] or None"""
        C, n = self._C, len(self.shards)
        self._x_keep, self._lg_keep = x, logits
        self._xs = (C.c_void_p * n)(*[x[l].data_ptr() for l in range(n)])
        self._lgs = None if logits is None else (C.c_void_p * n)(*[logits[l].data_ptr() for l in range(n)])

    def step(self):
        from .redcuda import RedcudaError
        st = torch.cuda.current_stream().cuda_stream
        if self._lib.redcuda_ep_step(self._h, self._layers, len(self.shards), self._xs, self._lgs, self._outs, st) != 1:
            raise RedcudaError(self._lib.redcuda_last_error().decode(errors="replace"))
        return self.out

    def layer_forward(self, l: int, x: torch.Tensor, logits: torch.Tensor | None = None) -> torch.Tensor:
        from .redcuda import RedcudaError
        st = torch.cuda.current_stream().cuda_stream
        if self._lib.redcuda_ep_layer_forward(self._h, self.shards[l].handle, x.data_ptr(), 0 if logits is None else logits.data_ptr(), self.out[l].data_ptr(), st) != 1:
            raise RedcudaError(self._lib.redcuda_last_error().decode(errors="replace"))
        return self.out[l]

    def close(self):
        if self._h:
            self.ctx.close()
            self._h = None
