"""Expert-parallel dispatch/combine on CPU ranks (gloo, world_size 2): the all-gather of rows,
the filter-mode local step (the CPU oracle stands in for it), the all-to-all back and the
rank-order combine."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, ret):
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path[:0] = [root, os.path.join(root, "muse-spark-kernels_b200")]
    from muse_moe_w4a16 import ep, inputs
    from oracle import moe_oracle as orc

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    H, I, E, k, T = 256, 256, 8, 3, 11
    w = inputs.make_weights(H, I, E, 4, "cpu", post_norm=True)          # same on every rank
    per = E // world
    local = {key: (v[rank * per:(rank + 1) * per] if key != "post_norm_w" else v) for key, v in w.items()}
    g = torch.Generator().manual_seed(50 + rank)
    x = torch.randn((T, H), generator=g).to(torch.bfloat16)
    ids, tw = orc.route_topk(torch.randn((T, E), generator=g), k)

    def experts(rows, rids, rw):
        return orc.moe_forward(rows, rids, rw, local, local_start=rank * per)

    out = ep.ep_step(x, ids, tw, experts, per)
    ref, parts = orc.moe_forward(x, ids, tw, w, return_parts=True)
    err = float((out.float() - parts["out_fp32"]).abs().max() / parts["out_fp32"].abs().max())
    # the rank-order combine reads a rank's rows only where the token routes to it
    mask = ep.route_mask(ids, world, per)
    ok_plan = bool(mask.any(0).all()) and int(mask.sum()) <= T * min(k, world)
    ret[rank] = (err, ok_plan)
    dist.barrier()
    dist.destroy_process_group()


def test_ep_step_two_cpu_ranks_matches_single_rank_oracle():
    world = 2
    port = _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    assert len(ret) == world
    for r in range(world):
        err, ok_plan = ret[r]
        assert ok_plan
        assert err <= 1e-2  # partial rows are rounded to bf16 before the rank-order sum


def test_combine_partials_skips_ranks_without_a_route():
    from muse_moe_w4a16 import ep

    g = torch.Generator().manual_seed(1)
    T, k, n, per, H = 40, 3, 4, 16, 32
    ids = torch.stack([torch.randperm(n * per, generator=g)[:k] for _ in range(T)])
    ids[5] = -1                                                  # a token without any route
    back = torch.randn((n, T, H), generator=g).to(torch.bfloat16)
    mask = ep.route_mask(ids, n, per)
    assert not bool(mask[:, 5].any())
    poisoned = back.clone()
    poisoned[~mask] = float("nan")                               # rows that must never be read
    out = ep.combine_partials(poisoned, ids, per)
    want = (back.float() * mask.unsqueeze(-1)).sum(0)
    assert torch.isfinite(out.float()).all()
    assert float((out.float() - want).abs().max()) <= 2e-2
    own = ep.combine_partials(poisoned, ids, per, self_rank=2, self_rows=back[2])
    assert torch.equal(own, out)


def _worker_peer_leaves(rank, world, port, ret):
    """Rank 1 leaves between steps (it never joins the exchange); rank 0 must get an error from its
    collective within the process group's time limit instead of waiting for ever."""
    import datetime
    import sys
    import time

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path[:0] = [root, os.path.join(root, "muse-spark-kernels_b200")]
    from muse_moe_w4a16 import ep

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))
    dist.barrier()                                   # both ranks are up
    if rank == 1:
        ret[rank] = "left"
        return                                       # gone before the step, nothing of it in flight
    T, H, k, per = 5, 64, 2, 4
    x = torch.zeros((T, H), dtype=torch.bfloat16)
    ids = torch.zeros((T, k), dtype=torch.int64)
    tw = torch.ones((T, k))
    t0 = time.time()
    try:
        ep.ep_step(x, ids, tw, lambda rows, rids, rw: rows, per)
        ret[rank] = "no error"
    except Exception as exc:                         # a time-out / connection error of the collective
        ret[rank] = ("error", type(exc).__name__, time.time() - t0)


def test_ep_step_surfaces_a_missing_rank_as_an_error():
    world = 2
    port = _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    ctx = mp.spawn(_worker_peer_leaves, args=(world, port, ret), nprocs=world, join=False)
    ctx.join(timeout=60)
    for proc in ctx.processes:
        if proc.is_alive():
            proc.terminate()
    assert ret.get(1) == "left"
    assert isinstance(ret.get(0), tuple) and ret[0][0] == "error", ret.get(0)
    assert ret[0][2] < 30.0


def test_exchange_deadline_raises_when_an_event_never_completes():
    """Host-side deadline of the GPU exchange, against a fake event: a peer that never answers leaves
    the last event of a step incomplete; wait_deadline must raise after the limit, not block."""
    import time

    from muse_moe_w4a16 import ep

    class NeverDone:
        def query(self):
            return False

    class DoneAfter:
        def __init__(self, n):
            self.n = n

        def query(self):
            self.n -= 1
            return self.n <= 0

    t0 = time.time()
    try:
        ep.wait_deadline(NeverDone(), 0.2, "step 7")
        raised = False
    except TimeoutError as exc:
        raised = "step 7" in str(exc)
    assert raised and 0.15 < time.time() - t0 < 5.0
    ep.wait_deadline(DoneAfter(3), 5.0, "step 8")    # completes: returns


def test_default_chunks_start_with_the_own_rank_and_end_with_one_rank():
    """chunk_sizes: every layout covers all source ranks; from four ranks on the default starts with the
    rank's own rows alone, ends with a single rank and takes at most two ranks at a time in between;
    explicit layouts are checked."""
    import pytest

    from muse_moe_w4a16 import ep

    for world in range(1, 17):
        sizes = ep.chunk_sizes(world)
        assert sum(sizes) == world and min(sizes) >= 1
        if world >= 4:
            assert sizes[0] == 1 and sizes[-1] == 1 and max(sizes) <= 2
    assert ep.chunk_sizes(8) == [1, 2, 2, 2, 1]
    assert ep.chunk_sizes(8, 4) == [2, 2, 2, 2]
    assert ep.chunk_sizes(8, [1, 3, 3, 1]) == [1, 3, 3, 1]
    with pytest.raises(ValueError):
        ep.chunk_sizes(8, 3)
    with pytest.raises(ValueError):
        ep.chunk_sizes(8, [4, 3])
