"""Expert parallelism for the routed-expert step: token dispatch and combine over all-to-all.

Rank r of n owns experts [r*E/n, (r+1)*E/n) (the reference's `local_start / local_count`
convention, muse_moe_w4a16/py/00_moe_w4a16.py:108-109; the reference itself only filters ids
and leaves the exchange to its caller, muse_moe_w4a16/cuda/moe.cu:347-350). Every rank holds
T tokens. One step:
  1. routing on the local tokens (ids, weights);
  2. dispatch: for each destination rank the tokens with at least one expert there, compacted
     in token order, travel with their ids/weights rows in equal-split buffers [n, C, ...],
     C = T (a token goes to a rank at most once, so nothing is ever dropped); unused rows carry
     ids = -1 and are ignored by the destination's sort. Equal splits need no host-side sizes:
     the step has no host synchronisation;
  3. the local expert step on the n*C received rows (kernel_fn with local_start), giving one
     partial row per received token;
  4. combine: the partial rows travel back the same way and each token sums its partial rows
     in rank order in FP32 (deterministic).
Collectives are torch.distributed all_to_all_single (NCCL on GPUs, over NVLink/NVSwitch; gloo in
the CPU tests). Remote data always lands in this rank's own memory before a kernel reads it.
"""
import torch
import torch.distributed as dist


def owner_rank(ids, experts_per_rank):
    return torch.div(ids, experts_per_rank, rounding_mode="floor")


def plan_dispatch(ids, n_ranks, experts_per_rank):
    """ids [T, k] (global) -> mask [n, T] (token t has a route on rank d), pos [n, T] (row of t in
    d's buffer), src [n, T] (token stored at row p of d's buffer; rows >= count hold token 0),
    count [n]."""
    T = ids.shape[0]
    dest = owner_rank(ids, experts_per_rank)                                  # [T, k]
    ranks = torch.arange(n_ranks, device=ids.device).view(n_ranks, 1, 1)
    mask = (dest.unsqueeze(0) == ranks).any(-1)                              # [n, T]
    pos = mask.long().cumsum(1) - 1                                          # [n, T]
    count = mask.sum(1)
    slot = torch.where(mask, pos, torch.full_like(pos, T))                   # row T = scratch row
    src = torch.zeros((n_ranks, T + 1), dtype=torch.long, device=ids.device)
    src.scatter_(1, slot, torch.arange(T, device=ids.device).expand(n_ranks, T))
    return mask, pos, src[:, :T].contiguous(), count


def _a2a(t, group):
    out = torch.empty_like(t)
    dist.all_to_all_single(out, t, group=group)
    return out


def ep_step(x, ids, weights, expert_fn, experts_per_rank, group=None):
    """x bf16 [T, H], ids int [T, k] (global ids), weights fp32 [T, k]. expert_fn(rows bf16
    [n*T, H], ids int32 [n*T, k], weights fp32 [n*T, k]) -> partial bf16 [n*T, H] computes this
    rank's experts (ids outside its range or negative are skipped). Returns out bf16 [T, H]."""
    n = dist.get_world_size(group)
    T, H = x.shape
    k = ids.shape[1]
    mask, pos, src, count = plan_dispatch(ids.long(), n, experts_per_rank)
    valid = torch.arange(T, device=x.device).view(1, T) < count.view(n, 1)   # [n, C]
    send_x = x[src]                                                          # [n, C, H]
    send_ids = torch.where(valid.unsqueeze(-1), ids.to(torch.int32)[src], torch.full((1,), -1, dtype=torch.int32,
                                                                                     device=x.device))
    send_w = weights.float()[src]
    recv_x = _a2a(send_x.contiguous(), group).view(n * T, H)
    recv_ids = _a2a(send_ids.contiguous(), group).view(n * T, k)
    recv_w = _a2a(send_w.contiguous(), group).view(n * T, k)
    partial = expert_fn(recv_x, recv_ids, recv_w)                            # [n*T, H] bf16
    back = _a2a(partial.view(n, T, H).contiguous(), group)                   # back[d, p]: rank d's partial of my row p
    return combine_partials(back, mask, pos)


def combine_partials(back, mask, pos):
    """out[t] = bf16(sum over ranks d, in rank order, of back[d, pos[d, t]] where mask[d, t]), FP32
    accumulation. On CUDA tensors this is one library kernel (msk_ep_combine); the torch loop
    below is the same arithmetic for the CPU (gloo) tests."""
    n, T, H = back.shape
    if back.is_cuda:
        import ctypes

        from . import _lib

        out = torch.empty((T, H), dtype=torch.bfloat16, device=back.device)
        m8 = mask.to(torch.uint8).contiguous()
        p64 = pos.contiguous()
        _lib.check(_lib.load().msk_ep_combine(_lib.ptr(back), _lib.ptr(m8), _lib.ptr(p64), _lib.ptr(out), n, T, T, H,
                                              ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)), "msk_ep_combine")
        return out
    out = torch.zeros((T, H), dtype=torch.float32, device=back.device)
    rows = torch.where(mask, pos, torch.zeros_like(pos))                     # [n, T]
    for d in range(n):                                                       # rank order, FP32
        out += back[d][rows[d]].float() * mask[d].unsqueeze(-1)
    return out.to(torch.bfloat16)



class EPModule:
    """prepare/kernel_fn for one rank of an expert-parallel group."""

    def __init__(self, local_weights, rank, world, n_experts, top_k, tokens_per_rank, group=None, **prep):
        import muse_moe_w4a16 as moe

        self.moe, self.rank, self.world, self.group = moe, rank, world, group
        self.n_experts, self.top_k, self.per_rank = n_experts, top_k, n_experts // world
        self.state = moe.prepare(local_weights, local_start=rank * self.per_rank, n_experts=n_experts, top_k=top_k,
                                 max_tokens=world * tokens_per_rank, **prep)

    def _experts(self, rows, ids, w):
        return self.moe.kernel_fn({"hidden_states": rows, "topk_ids": ids, "topk_weights": w}, self.state)

    def route(self, logits):
        import ctypes
        from . import _lib

        st, T = self.state, logits.shape[0]
        ids = torch.empty((T, self.top_k), dtype=torch.int32, device=logits.device)
        tw = torch.empty((T, self.top_k), dtype=torch.float32, device=logits.device)
        _lib.check(st["lib"].lib.msk_moe_route(ctypes.byref(st["cfg"]), _lib.ptr(logits), _lib.ptr(st["route_bias"]),
                                               _lib.ptr(ids), _lib.ptr(tw), T,
                                               ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)), "msk_moe_route")
        return ids, tw

    def kernel_fn(self, data):
        x = data["hidden_states"]
        if data.get("topk_ids") is not None:
            ids, tw = data["topk_ids"], data["topk_weights"]
        else:
            ids, tw = self.route(data["router_logits"].float().contiguous())
        return ep_step(x, ids, tw, self._experts, self.per_rank, self.group)


def bench_ep(args, spec, dev, rank, world, metric, unit, clock_sampler_cls, load_peaks):
    """The --gpus N > 1 arm of bench.py: config 4 (H7168 I2048 E256 top-8, T = 4096 per GPU)."""
    import json

    from . import inputs

    s = inputs.SHAPES[spec["shape"]]
    H, I, E, k, T = s["H"], s["I"], s["E"], s["k"], spec["T"]
    per = E // world
    weights = inputs.make_weights_random_bytes(H, I, per, 1000 + rank, dev)
    mod = EPModule(weights, rank, world, E, k, T)
    del weights
    torch.cuda.empty_cache()
    pool = [inputs.make_inputs(spec["shape"], T, 17 * rank + i, dev)[0] for i in range(4)]
    host_pool = [{"hidden_states": d["hidden_states"].cpu().pin_memory(),
                  "router_logits": d["router_logits"].cpu().pin_memory()} for d in pool]
    sampler = clock_sampler_cls(dev.index)
    sampler.start()

    def run(n, e2e):
        xd = torch.empty((T, H), dtype=torch.bfloat16, device=dev)
        ld = torch.empty((T, E), dtype=torch.float32, device=dev)
        out_h = torch.empty((T, H), dtype=torch.bfloat16).pin_memory()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(n):
            if e2e:
                hp = host_pool[i % len(pool)]
                xd.copy_(hp["hidden_states"], non_blocking=True)
                ld.copy_(hp["router_logits"], non_blocking=True)
                o = mod.kernel_fn({"hidden_states": xd, "router_logits": ld})
                out_h.copy_(o, non_blocking=True)
            else:
                mod.kernel_fn(pool[i % len(pool)])
        e1.record()
        torch.cuda.synchronize()
        dist.barrier()
        t = torch.tensor([e0.elapsed_time(e1)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    run(max(args.warmup, 3), False)
    ms = run(args.steps, False)
    run(max(args.warmup, 3), True)
    ms_e2e = run(args.steps, True)
    clocks = sampler.stop()
    from . import read_status

    status = torch.tensor([read_status(mod.state)], device=dev)
    dist.all_reduce(status, op=dist.ReduceOp.MAX)
    if int(status.item()) != 0:
        raise RuntimeError("device status word is non-zero on some rank")
    if rank == 0:
        peaks = load_peaks()
        flops = inputs.algorithmic_flops(H, I, T * k * world) * args.steps
        line = {
            "metric": metric, "value": T * world * args.steps / (ms * 1e-3), "unit": unit, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 x nvfp4 -> fp32 acc",
            "data": "synthetic",
            "config": {"workload": spec["name"], "tokens_per_gpu": T, "hidden": H, "inter": I, "experts": E,
                       "top_k": k, "parallelism": f"ep{world}", "l2": "inputs and weights exceed L2 (792 MB of weights per rank at 8 ranks)",
                       "dispatch": "all_to_all_single, equal splits C = T"},
            "e2e": {"value": T * world * args.steps / (ms_e2e * 1e-3), "unit": unit,
                    "h2d_bytes_per_step": (T * H * 2 + T * E * 4) * world, "d2h_bytes_per_step": T * H * 2 * world,
                    "ms_per_step": ms_e2e / args.steps},
            "gpu_launches": 5 * args.steps * world,
            "roofline": {"bound": "tensor", "achieved": flops / world / (ms * 1e-3) / 1e12,
                         "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
                         "frac": flops / world / (ms * 1e-3) / 1e12 / peaks["bf16_tflops_sustained"], "traffic": None,
                         "kernel": "whole EP step per GPU (GEMMs + all-to-all)",
                         "peak_source": peaks["source"] + " (sustained)"},
            "cpu_baseline": None,
            "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    dist.barrier()
    dist.destroy_process_group()
