"""Expert-parallel dispatch/combine host logic over gloo, world sizes 2 and 4, on CPU.

The expert FFN is replaced by a deterministic CPU stand-in so that the test
checks what the exchange must guarantee: every (token, slot) routing reaches
the rank that owns its expert, its result returns to the token's home rank in
(t, j) order, and the combined output equals the single-rank result exactly.
"""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from apus_b200.moe import ExpertParallelMoe, dispatch_plan, owner_ranks

E, TOPK, DIM = 8, 3, 16


def fake_route(x, ids):
    g = torch.Generator().manual_seed(int(x.abs().sum().item() * 1000) % 100000)
    s = x.shape[0]
    idx = torch.stack([torch.randperm(E, generator=g)[:TOPK] for _ in range(s)] or
                      [torch.zeros(TOPK, dtype=torch.int64)])[:s].to(torch.int32)
    wgt = torch.rand(s, TOPK, generator=g)
    return idx, wgt


def fake_expert(rows, eids):
    return rows * (eids.to(rows.dtype)[:, None] + 1.0) + 0.25


def fake_combine(eo, wgt, shared):
    s = wgt.shape[0]
    y = torch.zeros(s, DIM)
    for j in range(TOPK):                      # slot order, like the CUDA combine
        y = y + wgt[:, j:j + 1] * eo.reshape(s, TOPK, DIM)[:, j]
    return y + shared


def make(rank, world, check_local=None, padded=False):
    lo, hi = rank * (E // world), (rank + 1) * (E // world)

    def experts(rows, eids):
        if check_local is not None:
            live = eids >= 0                   # -1 = unused slot of the padded exchange
            assert bool(((eids[live] >= lo) & (eids[live] < hi)).all()), "routing reached the wrong rank"
        return fake_expert(rows, eids)
    return ExpertParallelMoe(E, TOPK, DIM, rank, world, experts_fn=experts, route_fn=fake_route,
                             shared_fn=lambda x: x * 0.5, combine_fn=fake_combine, padded=padded)


def worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.manual_seed(100 + rank)
    x = torch.randn(5 + rank, DIM)             # ragged batch sizes across ranks
    out = make(rank, world, check_local=True).forward(x)
    ref = make(0, 1).forward(x)                # same tokens, all experts local
    q.put((rank, bool(torch.equal(out, ref))))
    # an empty batch on one rank must not deadlock the exchange
    x0 = torch.randn(0 if rank == 1 else 3, DIM)
    out0 = make(rank, world).forward(x0)
    q.put((rank, out0.shape[0] == x0.shape[0]))
    # fixed-shape exchange (equal batches): same result as a single rank, bit for bit
    xp = torch.randn(6, DIM)
    outp = make(rank, world, check_local=True, padded=True).forward(xp)
    q.put((rank, bool(torch.equal(outp, make(0, 1).forward(xp)))))
    dist.destroy_process_group()


def test_dispatch_plan_groups_by_owner():
    idx = torch.tensor([[0, 5, 7], [3, 4, 1]])
    order, counts = dispatch_plan(idx, E, 2)
    assert counts.tolist() == [3, 3]
    dest = owner_ranks(idx.reshape(-1)[order], E, 2)
    assert dest.tolist() == [0, 0, 0, 1, 1, 1]
    assert order.tolist() == [0, 3, 5, 1, 2, 4]          # stable within a destination


def run_world(world):
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
        assert p.exitcode == 0
    res = [q.get(timeout=10) for _ in range(3 * world)]
    assert all(ok for _, ok in res), res


def test_expert_parallel_exchange_world2():
    run_world(2)


def test_expert_parallel_exchange_world4():
    """Four ranks of two experts each: the partition, the padded slots and the way back
    are the same code at 4 and 8 ranks as at 2."""
    run_world(4)
