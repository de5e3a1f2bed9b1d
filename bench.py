"""Benchmark of the routed-expert step (muse_moe_w4a16) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload decode|sweepT<n>|prefill|ep]
                    [--impl reference]

One JSON line on stdout. A step is one routed-expert pass (top-k routing, sort, gate/up GEMM +
SwiGLU, down GEMM, combine) over one batch of seeded synthetic input. Default workload at one
GPU: the T=1 decode configuration (H=4096, I=1536, E=128, top-8, uniform router logits).
  value      tokens/s, device-timed (CUDA events around CUDA-graph replays), inputs resident in HBM
  e2e        tokens/s through kernel_fn with pinned host inputs: H2D copies, launches, D2H of `out`
  roofline   dominant kernel (gate/up GEMM): algorithmic bytes or flops / its mean event-timed duration
  cpu_baseline  the CPU oracle (PyTorch eager on the host cores) on a bounded sample of the same inputs
L2 is flushed (a 256 MiB write) before every timed step, outside the timed interval, and the
steps cycle through a pool of different routings.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path[:0] = [ROOT, os.path.join(ROOT, "muse-spark-kernels_b200")]

METRIC = "routed_expert_tokens_per_s"
UNIT = "tokens/s"
POOL = 8  # distinct seeded inputs cycled through


def workload_spec(name, n_gpus):
    if name == "auto":
        name = "decode" if n_gpus == 1 else "ep"
    if name == "decode":
        return dict(name="decode_T1_H4096_I1536_E128_top8", shape="decode", T=1)
    if name.startswith("sweepT"):
        T = int(name[6:])
        return dict(name=f"sweep_T{T}_H4096_I1536_E128_top8", shape="sweep", T=T)
    if name == "prefill":
        return dict(name="prefill_T8192_H4096_I1536_E128_top8_zipf1.2", shape="prefill", T=8192)
    if name == "ep":
        return dict(name=f"ep{n_gpus}_T4096perGPU_H7168_I2048_E256_top8", shape="ep", T=4096)
    raise SystemExit(f"unknown workload {name}")


class ClockSampler:
    """Samples nvidia-smi SM clocks and throttle reasons while the timed regions run."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.stop_flag, self.thread = index, [], threading.Event(), None

    def _run(self):
        while not self.stop_flag.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5).stdout
                parts = [p.strip() for p in out.strip().split(",")]
                if len(parts) >= 7:
                    self.rows.append(parts)
            except Exception:
                pass
            self.stop_flag.wait(0.1)

    def start(self):
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()

    def stop(self):
        self.stop_flag.set()
        if self.thread:
            self.thread.join(timeout=6)
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm = [float(r[0]) for r in self.rows]
        reasons = set()
        for r in self.rows:
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": float(self.rows[0][1]), "reasons": sorted(reasons),
                "samples": len(sm)}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def cpu_oracle_run(spec, steps, sample_tokens=None, seed=0):
    """Times the CPU oracle (PyTorch eager + numpy dequant on the host cores) on a bounded sample:
    the touched experts of `steps` seeded inputs of the workload, capped at sample_tokens tokens."""
    import torch
    from muse_moe_w4a16 import inputs
    from oracle import moe_oracle as orc

    s = inputs.SHAPES[spec["shape"]]
    H, I, E, k = s["H"], s["I"], s["E"], s["k"]
    T = spec["T"] if sample_tokens is None else min(spec["T"], sample_tokens)
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    # weights only for the experts the sample touches (generated lazily, outside the timed part)
    cache = {}
    times = []
    for i in range(steps):
        data, _ = inputs.make_inputs(spec["shape"], T, seed + i, "cpu")
        ids, tw = orc.route_topk(data["router_logits"], k) if "router_logits" in data else (None, None)
        touched = sorted(set(ids.flatten().tolist()))
        for e in touched:
            if e not in cache:
                cache[e] = inputs.make_weights_random_bytes(H, I, 1, 1000 + e, "cpu")
        # dense local table over the touched experts only
        remap = {e: j for j, e in enumerate(touched)}
        lids = torch.tensor([[remap[int(v)] for v in row] for row in ids.tolist()], dtype=torch.int32)
        w = {key: torch.cat([cache[e][key] for e in touched]) for key in ("w13", "w13_sf", "w13_gs", "w2", "w2_sf", "w2_gs")}
        t0 = time.perf_counter()
        ids2, tw2 = orc.route_topk(data["router_logits"], k)
        orc.moe_forward(data["hidden_states"], lids, tw2, w)
        times.append(time.perf_counter() - t0)
        if sum(times) > 25.0:
            break
    tot = sum(times)
    return {"value": T * len(times) / tot, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"{len(times)} step(s) of T={T} tokens, touched experts only, PyTorch-eager CPU oracle "
                      f"(numpy NVFP4 dequant + fp32 matmul), {tot:.2f} s"}, tot / len(times)


def cpu_sample_tokens(spec):
    """Tokens of the bounded CPU sample: the cost is the dequantisation of the touched experts, so
    the sample is capped where it touches about 2.4e9 weights (64 tokens at H4096 I1536, 8 at
    H7168 I2048 E256): some tens of seconds per step on the host cores."""
    from muse_moe_w4a16 import inputs

    s = inputs.SHAPES[spec["shape"]]
    per_expert = 3 * s["I"] * s["H"]
    cap = 64 if per_expert <= 20e6 else 8
    return cap if spec["T"] > cap else None


def run_reference(args, spec):
    """--impl reference: the reference has no CPU implementation of this op and its CUDA kernel is
    sm_90a-only, so the arm times the CPU restatement of the reference math (oracle/) on the host
    cores, on a bounded sample of the same workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sample_tokens = cpu_sample_tokens(spec)
    steps = max(1, min(args.steps, 3))
    for _ in range(min(args.warmup, 1)):
        cpu_oracle_run(spec, 1, sample_tokens, seed=100)
    base, sec_per_step = cpu_oracle_run(spec, steps, sample_tokens)
    line = {"impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus,
            "steps": steps, "warmup": min(args.warmup, 1), "ms_per_step": sec_per_step * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 x nvfp4 -> fp32 acc",
            "data": "synthetic", "config": {"workload": spec["name"]}, "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def run_gpu(args, spec):
    import torch
    import torch.distributed as dist
    import muse_moe_w4a16 as moe
    from muse_moe_w4a16 import inputs

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    s = inputs.SHAPES[spec["shape"]]
    H, I, E, k, T = s["H"], s["I"], s["E"], s["k"], spec["T"]
    if world > 1:
        from muse_moe_w4a16 import ep
        return ep.bench_ep(args, spec, dev, rank, world, METRIC, UNIT, ClockSampler, load_peaks)

    if args.experts:
        # a smaller instance of the same kernels: fewer experts resident, same per-expert shapes
        s = dict(s, E=args.experts)
        inputs.SHAPES[spec["shape"]] = s
        E = args.experts
        spec = dict(spec, name=spec["name"] + f"_E{E}resident")
    peaks = load_peaks()
    weights = inputs.make_weights(H, I, E, 0, dev)
    state = moe.prepare(weights, n_experts=E, top_k=k, max_tokens=T, token_tile=args.token_tile)
    del weights
    torch.cuda.empty_cache()
    if args.profile_only:
        flush = torch.empty(64 * 1024 * 1024, dtype=torch.int32, device=dev)
        for i in range(max(args.warmup, 1) + args.steps):
            data, _ = inputs.make_inputs(spec["shape"], T, i % POOL, dev)
            flush.zero_()
            moe.kernel_fn(data, state)
        torch.cuda.synchronize()
        print(json.dumps({"profile_only": spec["name"], "plan": moe.plan(state, T), "status": moe.read_status(state)}))
        return
    pool, host_pool = [], []
    for i in range(POOL):
        data, _ = inputs.make_inputs(spec["shape"], T, i, dev)
        pool.append(data)
        host_pool.append({"hidden_states": data["hidden_states"].cpu().pin_memory(),
                          "router_logits": data["router_logits"].cpu().pin_memory()})
    flush = torch.empty(64 * 1024 * 1024, dtype=torch.int32, device=dev)  # 256 MiB > 126 MB of L2

    # touched experts / routed pairs of each pooled input (host side, outside any timed region)
    touched = []
    for data in pool:
        _, ids, _ = moe.kernel_fn(data, state, return_routing=True)
        touched.append(int(torch.unique(ids).numel()))
    torch.cuda.synchronize()
    if moe.read_status(state) != 0:
        raise RuntimeError("device status word is non-zero after warm-up")

    # CUDA graphs: one per pooled input
    graphs, outs = [], []
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for data in pool:
            moe.kernel_fn(data, state)
    torch.cuda.current_stream().wait_stream(side)
    for data in pool:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            o = moe.kernel_fn(data, state)
        graphs.append(g)
        outs.append(o)

    sampler = ClockSampler(local_rank)
    sampler.start()

    def timed_graph_steps(n):
        evs = []
        for i in range(n):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            graphs[i % POOL].replay()
            e1.record()
            evs.append((e0, e1))
        torch.cuda.synchronize()
        return [a.elapsed_time(b) for a, b in evs]

    timed_graph_steps(max(args.warmup, 3))
    torch.cuda.synchronize()
    step_ms = timed_graph_steps(args.steps)
    total_ms = sum(step_ms)

    # end to end with host buffers through the module's graphed step (the decode layer's way of calling it):
    # pinned host inputs -> static device buffers, graph replay, output back to pinned host memory
    step = moe.GraphedStep(state, pool[0])
    out_h = torch.empty((T, H), dtype=torch.bfloat16).pin_memory()

    def e2e_steps(n):
        evs = []
        for i in range(n):
            flush.zero_()
            hp = host_pool[i % POOL]
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            o = step(hp)
            out_h.copy_(o, non_blocking=True)
            e1.record()
            evs.append((e0, e1))
            if i % 64 == 63:
                torch.cuda.synchronize()
        torch.cuda.synchronize()
        return [a.elapsed_time(b) for a, b in evs]

    e2e_steps(max(args.warmup, 3))
    e2e_ms = e2e_steps(args.steps)

    # dominant kernel, event-timed inside the step
    n_prof = max(3, min(args.steps, 200))
    k_ms = [0.0, 0.0, 0.0, 0.0]
    for i in range(n_prof + 3):
        flush.zero_()
        _, ms = moe.kernel_fn_timed(pool[i % POOL], state)
        if i >= 3:
            k_ms = [a + b for a, b in zip(k_ms, ms)]
    k_ms = [v / n_prof for v in k_ms]
    clocks = sampler.stop()
    if moe.read_status(state) != 0:
        raise RuntimeError("device status word is non-zero after the timed region")

    mean_touched = sum(touched[i % POOL] for i in range(n_prof)) / n_prof
    R = T * k
    plan = moe.plan(state, T)
    hbm_bound = T <= 1024
    fused = plan[0] == 8   # the single-launch kernel for up to 8 tokens: it is the whole step
    if fused:
        alg = sum(inputs.algorithmic_bytes(H, I, E, k, T, touched[i % POOL]) for i in range(n_prof)) / n_prof
        achieved = alg / (k_ms[1] * 1e-3) / 1e9
        roof = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"], "traffic": None, "kernel": "moe_small_kernel (whole step)",
                "peak_source": peaks["source"] + " (burst copy)"}
    elif hbm_bound:
        # gate/up GEMM: touched experts' W13 tiles + the x rows it gathers + the inter rows it writes
        alg13 = mean_touched * (2 * I * H * 0.5625 + 4) + 2.0 * T * H + 2.0 * R * I
        achieved = alg13 / (k_ms[1] * 1e-3) / 1e9
        # DRAM traffic per launch: the ncu capture of this kernel on a 32-expert case read and
        # wrote 1.015 x its algorithmic bytes; weights dominate both, so it scales with the touched experts
        roof = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"], "traffic": alg13 * NCU_TRAFFIC_RATIO_GATE_UP,
                "traffic_source": "ncu dram bytes of the 32-expert T=64 capture / its algorithmic bytes (1.015), scaled",
                "kernel": "moe_gemm_kernel<N,0> (gate/up)", "peak_source": peaks["source"] + " (burst copy)"}
    else:
        fl13 = 2.0 * R * 2 * I * H
        achieved = fl13 / (k_ms[1] * 1e-3) / 1e12
        roof = {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
                "frac": achieved / peaks["bf16_tflops_sustained"], "traffic": None,
                "kernel": "moe_gemm_kernel<N,0> (gate/up)", "peak_source": peaks["source"] + " (sustained)"}
    step_bytes = sum(inputs.algorithmic_bytes(H, I, E, k, T, touched[i % POOL]) for i in range(args.steps))
    step_flops = inputs.algorithmic_flops(H, I, R) * args.steps
    cpu_base, _ = cpu_oracle_run(spec, 2, cpu_sample_tokens(spec))

    h2d = T * H * 2 + T * E * 4
    d2h = T * H * 2
    line = {
        "metric": METRIC, "value": T * args.steps / (total_ms * 1e-3), "unit": UNIT, "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": total_ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16 x nvfp4 -> fp32 acc", "data": "synthetic",
        "config": {"workload": spec["name"], "tokens": T, "hidden": H, "inter": I, "experts": E, "top_k": k,
                   "l2": "flushed by a 256 MiB write before every timed step", "cuda_graph": True,
                   "token_tile": plan[0], "split_k13": plan[1], "split_k2": plan[2], "ctas": plan[3],
                   "touched_experts_mean": mean_touched},
        "e2e": {"value": T * args.steps / (sum(e2e_ms) * 1e-3), "unit": UNIT, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": sum(e2e_ms) / args.steps},
        # per step: fused top-k + sort | top-k, sort (three launches from 16384 entries on), F16 row copy;
        # two GEMMs; combine
        "gpu_launches": (1 if fused else 4 if T <= 32 else 6 + (2 if T * k >= 16384 else 0)) * args.steps,
        "roofline": roof,
        "step_roofline": {"hbm_frac": step_bytes / (total_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                          "tensor_frac": step_flops / (total_ms * 1e-3) / 1e12 / peaks["bf16_tflops_sustained"],
                          "algorithmic_bytes_per_step": step_bytes / args.steps},
        "kernel_ms": {"sort": k_ms[0], "gemm_gate_up": k_ms[1], "gemm_down": k_ms[2], "combine": k_ms[3]},
        "cpu_baseline": cpu_base,
        "clocks": clocks,
    }
    print(json.dumps(line), flush=True)


NCU_TRAFFIC_RATIO_GATE_UP = 1.015   # ncu: DRAM bytes read + written / algorithmic bytes, gate/up kernel, 32-expert T = 64 case


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--workload", default="auto")
    ap.add_argument("--experts", type=int, default=0, help="resident experts (smaller case for profiler captures)")
    ap.add_argument("--ep-chunks", type=int, default=0, help="expert-parallel runs: chunks of source ranks (0 = default)")
    ap.add_argument("--token-tile", type=int, default=0, help="force a kernel: 16/32/64/128, 8 = single-launch kernel")
    ap.add_argument("--profile-only", action="store_true", help="run warmup+steps eager steps and exit (for ncu)")
    args = ap.parse_args()
    spec = workload_spec(args.workload, args.gpus)
    if args.impl == "reference":
        run_reference(args, spec)
    else:
        run_gpu(args, spec)


if __name__ == "__main__":
    main()
