"""Expert-parallel execution of the routed-expert step across the GPUs of one box.

The reference is single-GPU (one context, one stream, engine/src/engine.rs:73-74); sharding is new here and is defined
by "same result as one GPU". Layout: rank r of G owns experts [r*E/G, (r+1)*E/G) (all three tensors) and routes its own
tokens. One exchange each way:

  dispatch  every routed (token, slot) pair goes to the rank that owns its expert, as the token's Q8_K row (4672 B
            instead of 16 KB of f32) plus (local expert id, router weight);
  combine   the owner returns the pair's down-projection row (f32 [n_embd]); the source sums a token's k rows in slot
            order, so the result does not depend on arrival order.

Two implementations of the same plan live here. ``ExpertParallelHandle`` is the product path: a thin caller of the C
ABI (``dsmoe_ep_init`` / ``dsmoe_moe_forward_ep``), where counting, placement, row gather, the NCCL exchanges, the
owner's compute and the slot sum all happen inside the library on one stream. ``ExpertParallelMoe`` expresses the plan
with ``torch.distributed.all_to_all_single`` and replaceable ``route_fn`` / ``expert_fn``: it runs on gloo without a
GPU, with the oracle standing in for the kernels, which is how the CPU tests check the plan itself (dispatch order,
replicas, combine positions) with two ranks.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

from .formats import Q8K_BYTES, QK_K


class ExpertParallelHandle:
    """Expert-parallel state of one rank behind the C ABI. ``kernels``: a MoeKernels created with the model's n_expert
    and top-k and max_tokens = the tokens this rank routes per call. The NCCL communicator is created inside the library
    from a unique id that rank 0 makes and ``torch.distributed`` (any backend) carries to the other ranks."""

    def __init__(self, kernels, rank: int, world: int, max_replicas: int = 0, recv_capacity_rows: int = 0, group=None):
        import ctypes as C

        self.k, self.rank, self.world, self.max_replicas = kernels, rank, world, max_replicas
        self.per_rank = kernels.cfg.n_expert // world
        lib = kernels.lib
        uid = torch.zeros(128, dtype=torch.uint8)
        if rank == 0:
            buf = (C.c_uint8 * 128)()
            kernels._check(lib.dsmoe_ep_get_unique_id(buf))
            uid = torch.tensor(list(buf), dtype=torch.uint8)
        if world > 1:
            dev = torch.device("cuda", kernels.device) if dist.get_backend(group) == "nccl" else torch.device("cpu")
            uid = uid.to(dev)
            dist.broadcast(uid, src=0, group=group)
            uid = uid.cpu()
        ids = (C.c_uint8 * 128)(*uid.tolist())
        kernels._check(lib.dsmoe_ep_init(kernels.h, ids, rank, world, max_replicas, recv_capacity_rows))

    def layer_register(self, layer: int, gate, up, down, layout: int):
        """The rank's shard [own experts | replicas], per_rank + max_replicas experts long, already in ``layout``."""
        import ctypes as C

        p = lambda t: C.c_void_p(t.data_ptr())
        self.k._check(self.k.lib.dsmoe_ep_layer_register(self.k.h, layer, p(gate), p(up), p(down), layout))

    def set_replicas(self, expert_ids):
        import ctypes as C

        arr = (C.c_int32 * len(expert_ids))(*[int(e) for e in expert_ids])
        self.k._check(self.k.lib.dsmoe_ep_set_replicas(self.k.h, arr, len(expert_ids)))

    def expert_counts(self, reset: bool = False) -> torch.Tensor:
        """Running selections per expert on this rank (int64 [n_expert], host)."""
        import ctypes as C

        out = torch.zeros(self.k.cfg.n_expert, dtype=torch.int64)
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        self.k._check(self.k.lib.dsmoe_ep_expert_counts(self.k.h, stream, C.c_void_p(out.data_ptr()), int(reset)))
        return out

    @property
    def combine_is_fused(self) -> bool:
        """True when the owner's down projection stores its rows straight into the source ranks' buffers (peer memory)."""
        return bool(self.k.lib.dsmoe_ep_combine_is_fused(self.k.h))

    def last_recv_rows(self) -> list:
        import ctypes as C

        arr = (C.c_int32 * self.world)()
        self.k._check(self.k.lib.dsmoe_ep_last_recv_rows(self.k.h, arr))
        return list(arr)

    def set_phase_events(self, events):
        import ctypes as C

        if not events:
            self.k._check(self.k.lib.dsmoe_ep_set_phase_events(self.k.h, None, 0))
            return
        arr = (C.c_void_p * 6)(*[C.c_void_p(e.cuda_event) for e in events])
        self.k._check(self.k.lib.dsmoe_ep_set_phase_events(self.k.h, arr, 6))

    def forward(self, layer: int, x, logits, out=None, selected_out=None, weights_out=None):
        import ctypes as C

        T = x.shape[0]
        if out is None:
            out = torch.empty((T, self.k.cfg.n_embd), dtype=torch.float32, device=x.device)
        p = lambda t: None if t is None else C.c_void_p(t.data_ptr())
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        self.k._check(self.k.lib.dsmoe_moe_forward_ep(self.k.h, stream, layer, p(x), p(logits), T, p(out), p(selected_out),
                                                     p(weights_out)))
        return out


@dataclass
class DispatchPlan:
    """Where each local pair goes. ``order`` lists local pair ids grouped by destination rank, ascending pair id inside
    a group (stable), ``send_counts[d]`` pairs go to rank d, ``recv_counts[s]`` pairs come from rank s."""
    order: torch.Tensor
    send_counts: list
    recv_counts: list


def make_plan(selected: torch.Tensor, n_expert: int, world: int, group=None, stay_home=None, rank: int = 0) -> DispatchPlan:
    """selected: int32 [T, k] global expert ids (negative ids go to expert 0, as the kernels clamp them).
    stay_home: bool [n_expert] or None; pairs of those experts are computed on the rank that routed them."""
    per_rank = n_expert // world
    e = selected.reshape(-1).clamp(min=0).to(torch.int64)
    dest = e // per_rank
    if stay_home is not None:
        dest = torch.where(stay_home[e], torch.full_like(dest, rank), dest)
    order = torch.sort(dest, stable=True).indices
    send = torch.bincount(dest, minlength=world).to(torch.int64)
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    return DispatchPlan(order, [int(v) for v in send.cpu()], [int(v) for v in recv.cpu()])


def _exchange(buf: torch.Tensor, send_counts, recv_counts, group=None) -> torch.Tensor:
    """all_to_all_single over the first dimension with the given row counts."""
    out = buf.new_empty((sum(recv_counts),) + tuple(buf.shape[1:]))
    dist.all_to_all_single(out, buf.contiguous(), output_split_sizes=list(recv_counts),
                           input_split_sizes=list(send_counts), group=group)
    return out


class ExpertParallelMoe:
    """One layer's routed experts sharded over the ranks of ``group``.

    route_fn(x, logits) -> (xq uint8 [T, n_embd/256, 292], selected int32 [T, k], weights f32 [T, k])
    expert_fn(xq_rows, local_expert int32 [R, 1], weights f32 [R, 1]) -> f32 [R, n_embd]   (k = 1 on the owner)
    sum_fn(rows f32 [T*k, n_embd], pos int32 [T*k], T) -> f32 [T, n_embd]: slot e of token t is rows[pos[t*k+e]],
        slots added in slot order (default: un-permute, then k torch additions)
    """

    def __init__(self, route_fn, expert_fn, n_expert: int, k: int, n_embd: int, group=None, sum_fn=None, replicated=None):
        """replicated: global ids of experts every rank holds a copy of (the hottest ones), or None. Their pairs are
        not dispatched: the routing rank computes them itself, with local expert id per_rank + position in the list.
        The owner's expert table is then [own shard | replicas in list order]."""
        self.route_fn, self.expert_fn, self.sum_fn = route_fn, expert_fn, sum_fn
        self.replicated = None if replicated is None or len(replicated) == 0 else [int(e) for e in replicated]
        self.n_expert, self.k, self.n_embd = n_expert, k, n_embd
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        assert n_expert % self.world == 0, "experts must divide evenly over the ranks"
        self.per_rank = n_expert // self.world
        self.last_plan = None

    def forward(self, x: torch.Tensor, logits: torch.Tensor, mark=None):
        """x f32 [T, n_embd], logits f32 [T, n_expert] (this rank's tokens). Returns (out f32 [T, n_embd], selected).
        ``mark(name)``, if given, is called at the phase boundaries (the bench records CUDA events there)."""
        mark = mark or (lambda name: None)
        T = x.shape[0]
        mark("start")
        xq, selected, weights = self.route_fn(x, logits)
        mark("route")
        stay_home = replica_slot = None
        if self.replicated is not None:
            stay_home = torch.zeros(self.n_expert, dtype=torch.bool, device=selected.device)
            replica_slot = torch.zeros(self.n_expert, dtype=torch.int64, device=selected.device)
            ids = torch.tensor(self.replicated, dtype=torch.int64, device=selected.device)
            stay_home[ids] = True
            replica_slot[ids] = torch.arange(len(self.replicated), dtype=torch.int64, device=selected.device)
        plan = make_plan(selected, self.n_expert, self.world, self.group, stay_home, self.rank)
        self.last_plan = plan
        mark("plan")
        pair_tok = plan.order // self.k
        # dispatch: Q8_K row of the pair's token; local expert id and router weight (as its bit pattern) in one
        # int32 [pairs, 2] message
        xq_rows = xq.reshape(T, (self.n_embd // QK_K) * Q8K_BYTES)[pair_tok]
        sel_flat = selected.reshape(-1).clamp(min=0)[plan.order]
        local_e = sel_flat.to(torch.int64) % self.per_rank
        if stay_home is not None:
            local_e = torch.where(stay_home[sel_flat.to(torch.int64)], self.per_rank + replica_slot[sel_flat.to(torch.int64)], local_e)
        meta = torch.stack((local_e.to(torch.int32),
                            weights.reshape(-1)[plan.order].contiguous().view(torch.int32)), dim=1)
        r_xq = _exchange(xq_rows, plan.send_counts, plan.recv_counts, self.group)
        r_meta = _exchange(meta, plan.send_counts, plan.recv_counts, self.group)
        r_e = r_meta[:, 0:1].contiguous()
        r_w = r_meta[:, 1:2].contiguous().view(torch.float32)
        mark("dispatch")
        # the owner's compute: every received row is one (token, slot) pair of one local expert
        if r_xq.shape[0]:
            rows = self.expert_fn(r_xq.reshape(r_xq.shape[0], self.n_embd // QK_K, Q8K_BYTES), r_e, r_w)
        else:
            rows = x.new_empty((0, self.n_embd))
        mark("experts")
        # combine: rows travel back along the same splits, land in dispatch order, are put back in pair order and
        # summed per token in slot order
        back = _exchange(rows, plan.recv_counts, plan.send_counts, self.group)
        mark("combine")
        if self.sum_fn is not None:
            # position of every pair's row in ``back``: the inverse of the dispatch order
            pos = torch.empty_like(plan.order)
            pos[plan.order] = torch.arange(plan.order.numel(), device=plan.order.device)
            out = self.sum_fn(back, pos.to(torch.int32), T)
            mark("sum")
            return out, selected
        pair_rows = torch.empty((T * self.k, self.n_embd), dtype=back.dtype, device=back.device)
        pair_rows[plan.order] = back
        pr = pair_rows.reshape(T, self.k, self.n_embd)
        out = torch.zeros((T, self.n_embd), dtype=back.dtype, device=back.device)
        for s in range(self.k):  # 0 + r0 + r1 + ..., the order of the reference's slot sum (moe.rs:937-968, 983-1005)
            out = out + pr[:, s]
        return out, selected


def gpu_functions(kernels_route, kernels_owner, layer: int = 0):
    """route_fn / expert_fn over the C ABI (``gpu_sum_function`` gives the matching sum_fn). ``kernels_route``: a MoeKernels with the model's k (router + Q8_K only);
    ``kernels_owner``: a MoeKernels created with n_expert = experts per rank and n_expert_used = 1, holding this rank's
    shard in ``layer``."""
    cfg = kernels_route.cfg

    def route_fn(x, logits):
        T = x.shape[0]
        dev = x.device
        probs = torch.empty((T, cfg.n_expert), dtype=torch.float32, device=dev)
        sel = torch.empty((T, cfg.n_expert_used), dtype=torch.int32, device=dev)
        w = torch.empty((T, cfg.n_expert_used), dtype=torch.float32, device=dev)
        xq = torch.empty((T, cfg.n_embd // QK_K, Q8K_BYTES), dtype=torch.uint8, device=dev)
        kernels_route.router_select_parallel(logits, None, None, None, probs, sel, w, 0, 0, T, 0, 0)
        kernels_route.q8k_quantize(x, xq, cfg.n_embd, T)
        return xq, sel, w

    def expert_fn(xq_rows, local_expert, weights):
        R = xq_rows.shape[0]
        out = torch.empty((R, cfg.n_embd), dtype=torch.float32, device=xq_rows.device)
        kernels_owner.expert_ffn(layer, xq_rows.contiguous(), local_expert.contiguous(), weights.contiguous(), R, out)
        return out

    return route_fn, expert_fn


def gpu_sum_function(kernels_route):
    """sum_fn over the C ABI: the slot-order sum kernel (engine/src/kernels/moe.rs:983)."""
    cfg = kernels_route.cfg

    def sum_fn(rows, pos, T):
        out = torch.empty((T, cfg.n_embd), dtype=torch.float32, device=rows.device)
        kernels_route.moe_sum_indexed(rows.contiguous(), pos.contiguous(), out, cfg.n_embd, cfg.n_expert_used, T)
        return out

    return sum_fn
