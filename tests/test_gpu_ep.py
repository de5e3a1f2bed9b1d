"""Expert parallelism on real GPUs (NCCL, 2 ranks): the EP step against the single-GPU step
with all experts resident. Skipped on boxes with fewer than two GPUs."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


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
    import muse_moe_w4a16 as moe
    from muse_moe_w4a16 import ep, inputs

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    H, I, E, k, T = 1024, 512, 16, 4, 97
    w = inputs.make_weights(H, I, E, 9, dev)                      # same seed on every rank
    per = E // world
    local = {key: v[rank * per:(rank + 1) * per].contiguous() for key, v in w.items()}
    full = moe.prepare(w, n_experts=E, top_k=k, max_tokens=T)
    errs, stats = [], []
    for transport, chunks in (("symm", 1), ("symm", 2), ("collective", None)):
        mod = ep.EPModule(local, rank, world, E, k, T, transport=transport, chunks=chunks)
        for step in range(3):                                     # both buffer parities and their reuse
            g = torch.Generator(device=dev).manual_seed(70 + rank + 10 * step)
            x = torch.randn((T, H), generator=g, device=dev).to(torch.bfloat16)
            logits = torch.randn((T, E), generator=g, device=dev)
            out = mod.kernel_fn({"hidden_states": x, "router_logits": logits})
            ref = moe.kernel_fn({"hidden_states": x, "router_logits": logits}, full)
            torch.cuda.synchronize()
            errs.append(float((out.float() - ref.float()).abs().max() / ref.float().abs().max()))
        stats.append(moe.read_status(mod.state))
    ret[rank] = (max(errs), max(stats), moe.read_status(full))
    dist.barrier()
    dist.destroy_process_group()


def test_ep_two_gpus_matches_single_gpu(cuda_dev):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    for r in range(world):
        err, s1, s2 = ret[r]
        assert s1 == 0 and s2 == 0
        assert err <= 1e-2
