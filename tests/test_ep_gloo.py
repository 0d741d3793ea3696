"""Expert-parallel dispatch / combine on two CPU ranks (gloo): the plan, the all-to-all exchanges and the slot-order
combine of deepseek_rs_b200/ep.py, with the oracle standing in for the kernels on each rank. The sharded result must
equal the single-rank oracle layer bit for bit, and the routing must be identical."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist

    import oracle
    from deepseek_rs_b200 import formats as F
    from deepseek_rs_b200.ep import ExpertParallelMoe

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    oracle.set_num_threads(2)
    n_e, n_embd, n_ff, k, T = 8, 512, 256, 3, 5 + rank  # ragged: ranks hold different token counts
    lw = F.ExpertLayer(seed=41, n_expert=n_e, n_embd=n_embd, n_ff=n_ff)
    per = n_e // world
    gsh = lw.gate.reshape(n_e, -1)[rank * per:(rank + 1) * per].reshape(-1)
    ush = lw.up.reshape(n_e, -1)[rank * per:(rank + 1) * per].reshape(-1)
    dsh = lw.down.reshape(n_e, -1)[rank * per:(rank + 1) * per].reshape(-1)
    rng = np.random.default_rng(100)  # same stream on both ranks; each takes its slice
    x_all = rng.standard_normal((11, n_embd)).astype(np.float32)
    lg_all = rng.standard_normal((11, n_e)).astype(np.float32)
    lg_all[0, :] = 0.5  # ties: lowest expert ids win on every rank alike
    lo = 0 if rank == 0 else 5
    x, lg = x_all[lo:lo + T], lg_all[lo:lo + T]

    def route_fn(xt, lt):
        _, sel, w = oracle.router_select(lt.numpy(), k=k)
        return torch.from_numpy(oracle.q8k_quantize(xt.numpy())), torch.from_numpy(sel), torch.from_numpy(w)

    def expert_fn(xq_rows, local_e, w):
        _, _, mid = oracle.gate_up_mid(gsh, ush, xq_rows.numpy(), local_e.numpy(), w.numpy(), n_ff, n_embd // 256)
        midq = oracle.q8k_quantize(mid)
        return torch.from_numpy(oracle.down(dsh, midq, local_e.numpy(), n_embd, n_ff // 256))

    ep = ExpertParallelMoe(route_fn, expert_fn, n_e, k, n_embd)
    out, sel = ep.forward(torch.from_numpy(x), torch.from_numpy(lg))
    ref_out, ref_sel, _ = oracle.moe_layer(x, lg, lw.gate, lw.up, lw.down, k=k, n_ff=n_ff)
    ok = bool(np.array_equal(out.numpy(), ref_out) and np.array_equal(sel.numpy(), ref_sel))
    sent = sum(ep.last_plan.send_counts)
    # a second step with no tokens on rank 1: empty sends and receives must not hang or mis-size anything
    T2 = 4 if rank == 0 else 0
    out2, _ = ep.forward(torch.from_numpy(x_all[:T2]), torch.from_numpy(lg_all[:T2]))
    if T2:
        ref2, _, _ = oracle.moe_layer(x_all[:T2], lg_all[:T2], lw.gate, lw.up, lw.down, k=k, n_ff=n_ff)
        ok = ok and bool(np.array_equal(out2.numpy(), ref2))
    else:
        ok = ok and out2.shape == (0, n_embd)
    # third step: experts 1 and 6 are replicated on both ranks (local ids per, per + 1); their pairs stay home and the
    # result is still the single-rank layer's
    rep = [6, 1]
    def shard_with(t):
        full = t.reshape(n_e, -1)
        return np.concatenate([full[rank * per:(rank + 1) * per], full[rep]]).reshape(-1)
    g3, u3, d3 = shard_with(lw.gate), shard_with(lw.up), shard_with(lw.down)

    def expert_fn3(xq_rows, local_e, w):
        _, _, mid = oracle.gate_up_mid(g3, u3, xq_rows.numpy(), local_e.numpy(), w.numpy(), n_ff, n_embd // 256)
        return torch.from_numpy(oracle.down(d3, oracle.q8k_quantize(mid), local_e.numpy(), n_embd, n_ff // 256))

    ep3 = ExpertParallelMoe(route_fn, expert_fn3, n_e, k, n_embd, replicated=rep)
    out3, _ = ep3.forward(torch.from_numpy(x), torch.from_numpy(lg))
    ok = ok and bool(np.array_equal(out3.numpy(), ref_out))
    home = int(np.isin(ref_sel, rep).sum())  # pairs that must not have left this rank
    ok = ok and ep3.last_plan.send_counts[rank] >= home
    q.put((rank, ok, sent, T * k))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_expert_parallel_two_ranks_matches_single_rank():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ok, sent, pairs in results:
        assert ok, f"rank {rank}: sharded result differs from the single-rank layer"
        assert sent == pairs  # every pair was dispatched exactly once


def test_peer_store_slots_equal_an_all_to_all():
    """The peer-store exchanges address the destination's buffer directly: send position i of rank r, lying in the
    segment for destination d, goes to slot recv_base[r][d] + (i - send_begin[r][d]) of rank d, with recv_base[r][d] =
    sum of M[s][d] over s < r (M[s][d] = rows rank s sends to rank d). This replays that arithmetic (csrc/ep.cu, the
    gather's EpPeerDst and the combine's EpRowMap) on random count matrices and checks it against what an all-to-all
    with the same splits delivers: every destination's slots are filled exactly once, grouped by source rank in rank
    order, in send order inside a group; and the return path lands every result row on the position it was sent from."""
    rng = np.random.default_rng(5)
    for world in (1, 2, 4, 8, 16):
        M = rng.integers(0, 50, size=(world, world))
        M[rng.integers(0, world), :] = 0  # a rank that sends nothing
        M[:, rng.integers(0, world)] = 0  # a rank that receives nothing
        send_end = np.cumsum(M, axis=1)                       # [r][d]: end of d's segment in r's send order
        send_begin = send_end - M
        recv_base = np.cumsum(M, axis=0) - M                  # [r][d]: first slot of r's segment at d
        recv = [[None] * int(M[:, d].sum()) for d in range(world)]
        for r in range(world):
            for i in range(int(M[r].sum())):
                d = 0
                while d + 1 < world and i >= send_end[r][d]:  # the kernels' linear search over destinations
                    d += 1
                slot = int(recv_base[r][d] + (i - send_begin[r][d]))
                assert recv[d][slot] is None
                recv[d][slot] = (r, i)
        for d in range(world):
            want = [(r, int(send_begin[r][d]) + j) for r in range(world) for j in range(int(M[r][d]))]
            assert recv[d] == want                            # = all_to_all_single with these splits
            seg_end = np.cumsum(M[:, d])                      # combine: received row j came from rank s, position ...
            for j, (r, i) in enumerate(recv[d]):
                s = 0
                while s + 1 < world and j >= seg_end[s]:
                    s += 1
                begin = int(seg_end[s] - M[s][d])
                dst_base = int(M[s][:d].sum())                # first slot of d's segment in s's send order
                assert (s, dst_base + (j - begin)) == (r, i)
