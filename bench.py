"""Benchmark of the routed-expert step (muse_moe_w4a16) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload auto|decode|sweepT<n>|prefill|ep]
                    [--no-sweep] [--impl reference]

One JSON line on stdout. A step is one routed-expert pass (top-k routing, sort, gate/up GEMM +
SwiGLU, down GEMM, combine) over one batch of seeded synthetic input.
  N = 1    headline workload: the T = 1 decode configuration (H4096 I1536 E128 top-8, uniform router
           logits); the line also carries `sweep`: the other points of the metric (T = 8 .. 256 with
           N(0,1) logits, and the T = 8192 Zipf-routed prefill), measured the same way on the same
           prepared weights with fewer steps each.
  N > 1    the expert-parallel configuration (H7168 I2048 E256 top-8, T = 4096 per GPU). Before the
           timing rank 0 also runs the same shape with all 256 experts on its one GPU: every rank checks
           its expert-parallel output against that (`ep_parity_max_rel`), and the line carries
           `single_gpu_same_shape_ms` and `scaling_efficiency` = that / the N-GPU step.
  value      tokens/s, device-timed (CUDA events around CUDA-graph replays), inputs resident in HBM
  e2e        tokens/s through the module's graphed step with pinned host inputs: H2D copy, launch,
             D2H of `out`; event-timed, with the host wall-clock time per step beside it
  roofline   dominant kernel: algorithmic bytes or flops / its mean event-timed duration
  cpu_baseline  the CPU oracle (PyTorch eager on the host cores) on a bounded sample of the same inputs
L2 is flushed before every timed step, outside the timed interval, by reading a 256 MiB buffer
(`--flush write` zeroes it instead: that leaves L2 full of dirty lines whose write-back competes
with the step; the reference sweeps by reading for that reason), and the steps cycle through a
pool of different routings.
"""
import argparse
import json
import math
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
DTYPE = "bf16 x nvfp4 -> fp32 acc"
POOL = 8  # distinct seeded inputs cycled through
SWEEP = ("sweepT8", "sweepT32", "sweepT64", "sweepT128", "sweepT256", "prefill")
HOST_MAPPED_MAX_TOKENS = 64   # up to here the end-to-end leg also tries the copy-free transport
NCU_TRAFFIC_RATIO = 1.015   # ncu: DRAM bytes read + written / algorithmic bytes of the weight-streaming GEMM kernel


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
        return self

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


# ------------------------------------------------------------------ CPU arm
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
    from muse_moe_w4a16 import inputs

    s = inputs.SHAPES[spec["shape"]]
    sample_tokens = cpu_sample_tokens(spec)
    steps = max(1, min(args.steps, 3))
    for _ in range(min(args.warmup, 1)):
        cpu_oracle_run(spec, 1, sample_tokens, seed=100)
    base, sec_per_step = cpu_oracle_run(spec, steps, sample_tokens)
    config = {"workload": spec["name"], "hidden": s["H"], "inter": s["I"], "experts": s["E"], "top_k": s["k"]}
    config["tokens_per_gpu" if spec["shape"] == "ep" else "tokens"] = spec["T"]
    line = {"impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus,
            "steps": steps, "warmup": min(args.warmup, 1), "ms_per_step": sec_per_step * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": DTYPE,
            "data": "synthetic", "config": config, "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------ one GPU, one workload
def measure(moe, inputs, state, spec, steps, warmup, peaks, dev, flush_fn, with_e2e=True):
    """Times one workload on a prepared state. Returns the dict that goes into the JSON line."""
    import torch

    s = inputs.SHAPES[spec["shape"]]
    H, I, E, k, T = s["H"], s["I"], s["E"], s["k"], spec["T"]
    pool, host_pool = [], []
    for i in range(POOL):
        data, _ = inputs.make_inputs(spec["shape"], T, i, dev)
        pool.append(data)
        if with_e2e:
            host_pool.append({"hidden_states": data["hidden_states"].cpu().pin_memory(),
                              "router_logits": data["router_logits"].cpu().pin_memory()})
    # touched experts of each pooled input (host side, outside any timed region)
    touched = []
    for data in pool:
        _, ids, _ = moe.kernel_fn(data, state, return_routing=True)
        touched.append(int(torch.unique(ids).numel()))
    torch.cuda.synchronize()
    if moe.read_status(state) != 0:
        raise RuntimeError("device status word is non-zero after warm-up")

    # CUDA graphs: one per pooled input
    graphs = []
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for data in pool:
            moe.kernel_fn(data, state)
    torch.cuda.current_stream().wait_stream(side)
    for data in pool:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            moe.kernel_fn(data, state)
        graphs.append(g)

    sampler = ClockSampler(dev.index or 0).start()

    def timed_graph_steps(n):
        evs = []
        for i in range(n):
            flush_fn()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            graphs[i % POOL].replay()
            e1.record()
            evs.append((e0, e1))
        torch.cuda.synchronize()
        return [a.elapsed_time(b) for a, b in evs]

    timed_graph_steps(max(warmup, 3))
    step_ms = timed_graph_steps(steps)
    total_ms = sum(step_ms)

    e2e = None
    if with_e2e:
        # end to end with host buffers through the module's graphed step (the decode layer's way of calling
        # it): pinned host inputs -> static device buffers, graph replay, output back to pinned host memory
        step = moe.GraphedStep(state, pool[0])
        out_h = torch.empty((T, H), dtype=torch.bfloat16).pin_memory()

        def e2e_steps(n):
            evs = []
            for i in range(n):
                flush_fn()
                hp = host_pool[i % POOL]
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                out_h.copy_(step(hp), non_blocking=True)
                e1.record()
                evs.append((e0, e1))
                if i % 64 == 63:
                    torch.cuda.synchronize()
            torch.cuda.synchronize()
            return [a.elapsed_time(b) for a, b in evs]

        def wall_steps(n):
            # what a caller that needs the result on the host feels: Python, staging copy, launch, D2H, sync
            ts = []
            for i in range(n):
                flush_fn()
                torch.cuda.synchronize()
                hp = host_pool[i % POOL]
                t0 = time.perf_counter()
                out_h.copy_(step(hp), non_blocking=True)
                torch.cuda.synchronize()
                ts.append((time.perf_counter() - t0) * 1e3)
            return ts

        e2e_steps(max(warmup, 3))
        e2e_ms = e2e_steps(steps)
        wall = wall_steps(min(steps, 100))
        e2e = {"value": T * steps / (sum(e2e_ms) * 1e-3), "unit": UNIT, "h2d_bytes_per_step": T * H * 2 + T * E * 4,
               "d2h_bytes_per_step": T * H * 2, "ms_per_step": sum(e2e_ms) / steps,
               "wall_ms_per_step": statistics.median(wall), "wall_value": T / (statistics.median(wall) * 1e-3),
               "transport": "pinned staging block -> one H2D copy -> graph replay -> D2H copy to pinned memory"}
        if T <= HOST_MAPPED_MAX_TOKENS:
            # the other transport: the kernels read the pinned host inputs and write the pinned host output
            # themselves (no copy launches); the same bytes cross PCIe inside the timed region
            hstep = moe.HostMappedStep(state, host_pool[0])   # raises (and the run with it) if it cannot be built:
            # a benchmark that silently dropped one of its two transports would not be the same benchmark

            def e2e_steps_mapped(n):
                evs = []
                for i in range(n):
                    flush_fn()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    hstep(host_pool[i % POOL])
                    e1.record()
                    evs.append((e0, e1))
                torch.cuda.synchronize()
                return [a.elapsed_time(b) for a, b in evs]

            def wall_steps_mapped(n):
                ts = []
                for i in range(n):
                    flush_fn()
                    torch.cuda.synchronize()
                    t0 = time.perf_counter()
                    hstep(host_pool[i % POOL])
                    hstep.done.synchronize()
                    ts.append((time.perf_counter() - t0) * 1e3)
                return ts

            e2e_steps_mapped(max(warmup, 3))
            m_ms = e2e_steps_mapped(steps)
            m_wall = wall_steps_mapped(min(steps, 100))
            mapped = dict(e2e, value=T * steps / (sum(m_ms) * 1e-3), ms_per_step=sum(m_ms) / steps,
                          wall_ms_per_step=statistics.median(m_wall), wall_value=T / (statistics.median(m_wall) * 1e-3),
                          transport="host-mapped: the kernels read the pinned host inputs and write the pinned host "
                                    "output over PCIe (HostMappedStep), no copy launches")
            # the faster transport is the module's answer at this size; the other is kept beside it
            if mapped["ms_per_step"] < e2e["ms_per_step"]:
                e2e, other = mapped, e2e
            else:
                other = mapped
            e2e["other_transport"] = {k2: other[k2] for k2 in ("transport", "value", "ms_per_step", "wall_ms_per_step")}

    # the kernels, event-timed one by one inside the step
    n_prof = max(3, min(steps, 200))
    k_ms = [0.0] * 5
    for i in range(n_prof + 3):
        flush_fn()
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
    one_launch = plan[1] == 0 and T <= 32 and R <= 256
    both_gemms = plan[1] == 4     # sort launch(es), both GEMMs in one launch, combine
    step_bytes = sum(inputs.algorithmic_bytes(H, I, E, k, T, touched[i % POOL]) for i in range(steps)) / steps
    step_flops = inputs.algorithmic_flops(H, I, R)
    if one_launch:
        alg = sum(inputs.algorithmic_bytes(H, I, E, k, T, touched[i % POOL]) for i in range(n_prof)) / n_prof
        achieved = alg / (k_ms[2] * 1e-3) / 1e9
        roof = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"], "traffic": alg * NCU_TRAFFIC_RATIO,
                "traffic_source": "ncu dram bytes of a weight-streaming GEMM capture / its algorithmic bytes (1.015), scaled",
                "kernel": "moe_gemm_kernel<N,2> (whole step in one launch)",
                "peak_source": peaks["source"] + " (burst copy)"}
    elif both_gemms:
        # both GEMMs in one launch: the touched experts' tiles of both, x read and converted, inter written and
        # read back, y written
        alg = mean_touched * (3 * I * H * 0.5625 + 8) + 4.0 * T * H + 4.0 * R * I + 4.0 * R * H
        achieved = alg / (k_ms[2] * 1e-3) / 1e9
        roof = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"], "traffic": alg * NCU_TRAFFIC_RATIO,
                "traffic_source": "ncu dram bytes of a weight-streaming GEMM capture / its algorithmic bytes (1.015), scaled",
                "kernel": "moe_gemm_kernel<N,2> (gate/up and down GEMM in one launch)",
                "peak_source": peaks["source"] + " (burst copy)"}
    elif T <= 1024:
        # gate/up GEMM: touched experts' W13 tiles + the x rows it gathers + the inter rows it writes
        alg13 = mean_touched * (2 * I * H * 0.5625 + 4) + 2.0 * T * H + 2.0 * R * I
        achieved = alg13 / (k_ms[2] * 1e-3) / 1e9
        roof = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"], "traffic": alg13 * NCU_TRAFFIC_RATIO,
                "traffic_source": "ncu dram bytes of the 32-expert T=64 capture / its algorithmic bytes (1.015), scaled",
                "kernel": "moe_gemm_kernel<N,0> (gate/up)", "peak_source": peaks["source"] + " (burst copy)"}
    else:
        fl13 = 2.0 * R * 2 * I * H
        achieved = fl13 / (k_ms[2] * 1e-3) / 1e12
        roof = {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
                "frac": achieved / peaks["bf16_tflops_sustained"], "frac_of_burst_peak": achieved / peaks["bf16_tflops"],
                "peak_burst": peaks["bf16_tflops"], "traffic": None,
                "kernel": "moe_gemm_kernel<N,0> (gate/up)", "peak_source": peaks["source"] + " (sustained; burst beside it)"}
    sec = total_ms / steps * 1e-3
    if one_launch:
        launches = 1
    elif plan[1] == 2 and T <= 32 and R <= 256:
        launches = 3      # row copy, gate/up kernel (routes, sorts), down kernel (combines)
    elif both_gemms:      # [top-k +] sort (one launch up to 32 tokens), both GEMMs, combine
        launches = 3 if T <= 32 else 4
    else:                 # [top-k +] sort (one launch up to 32 tokens, three from 16384 entries), row copy, two GEMMs, combine
        launches = 4 if T <= 32 else 6 + (2 if T * k >= 16384 else 0)
    return {
        "workload": spec["name"], "tokens": T, "steps": steps, "ms_per_step": total_ms / steps,
        "value": T / sec, "unit": UNIT,
        "plan": {"token_tile": plan[0], "path": plan[1], "flat_shares": plan[2], "ctas": plan[3],
                 "touched_experts_mean": mean_touched},
        "gpu_launches_per_step": launches,
        "roofline": roof,
        "step_roofline": {"hbm_frac": step_bytes / sec / 1e9 / peaks["hbm_gbs"],
                          "tensor_frac": step_flops / sec / 1e12 / peaks["bf16_tflops_sustained"],
                          "tensor_frac_of_burst_peak": step_flops / sec / 1e12 / peaks["bf16_tflops"],
                          "algorithmic_bytes_per_step": step_bytes, "algorithmic_flops_per_step": step_flops},
        "kernel_ms": {"route_sort": k_ms[0], "row_copy": k_ms[1], "gemm_gate_up": k_ms[2], "gemm_down": k_ms[3],
                      "combine": k_ms[4]},
        "e2e": e2e, "clocks": clocks,
    }


def measure_rotating(moe, inputs, states, spec, steps, warmup, peaks, dev):
    """The same step timed the other way the timing rules allow: no L2 sweep, inputs larger than L2.
    Consecutive steps run on different weight sets (len(states) sets of all experts, each a separate
    allocation) and different pooled inputs, so every weight byte a step reads was last read at least
    len(states) - 1 steps earlier, with more than L2's size of other weights streamed in between; the
    kernels' code, a few hundred KB shared by all steps, stays in L2, as it does when a model runs this
    layer once per MoE layer. Steps are CUDA-graph replays issued back to back; the time is first event
    to last event over the steps, so launch gaps count."""
    import torch

    s = inputs.SHAPES[spec["shape"]]
    H, I, E, k, T = s["H"], s["I"], s["E"], s["k"], spec["T"]
    pool = [inputs.make_inputs(spec["shape"], T, i, dev)[0] for i in range(POOL)]
    n_graphs = len(states) * POOL // math.gcd(len(states), POOL)   # step i: weight set i % R, input i % POOL
    touched = []
    for i in range(n_graphs):
        _, ids, _ = moe.kernel_fn(pool[i % POOL], states[i % len(states)], return_routing=True)
        touched.append(int(torch.unique(ids).numel()))
    torch.cuda.synchronize()
    graphs = []
    for i in range(n_graphs):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            moe.kernel_fn(pool[i % POOL], states[i % len(states)])
        graphs.append(g)
    per_step_bytes = [inputs.algorithmic_bytes(H, I, E, k, T, t) for t in touched]
    min_between = min(sum(per_step_bytes[(i + j) % n_graphs] for j in range(1, len(states))) for i in range(n_graphs))

    def run(n):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(n):
            graphs[i % n_graphs].replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)

    run(max(warmup, 3) + n_graphs)
    ms = run(steps) / steps
    if any(moe.read_status(st) != 0 for st in states):
        raise RuntimeError("device status word is non-zero after the rotating-weights run")
    step_bytes = sum(per_step_bytes[i % n_graphs] for i in range(steps)) / steps
    return {"ms_per_step": ms, "value": T / (ms * 1e-3), "unit": UNIT, "steps": steps, "weight_sets": len(states),
            "hbm_frac": step_bytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
            "weight_bytes_streamed_before_a_set_is_reused": min_between,
            "l2": "not swept: consecutive steps use different weight sets and inputs (inputs larger than L2); "
                  "back-to-back CUDA-graph replays, first event to last event"}


def run_gpu(args, spec):
    import torch
    import muse_moe_w4a16 as moe
    from muse_moe_w4a16 import _lib, inputs

    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        return run_ep(args, spec, dev)

    s = inputs.SHAPES[spec["shape"]]
    if args.experts:
        # a smaller instance of the same kernels: fewer experts resident, same per-expert shapes
        for key in ("decode", "sweep", "prefill"):
            inputs.SHAPES[key] = dict(inputs.SHAPES[key], E=args.experts)
        s = inputs.SHAPES[spec["shape"]]
        spec = dict(spec, name=spec["name"] + f"_E{args.experts}resident")
    H, I, E, k, T = s["H"], s["I"], s["E"], s["k"], spec["T"]
    peaks = load_peaks()
    sweep_specs = []
    if args.workload == "auto" and not args.no_sweep and not args.profile_only:
        sweep_specs = [workload_spec(w, 1) for w in SWEEP]
        if args.experts:
            sweep_specs = [dict(w, name=w["name"] + f"_E{args.experts}resident") for w in sweep_specs]
    max_tokens = max([T] + [w["T"] for w in sweep_specs])
    weights = inputs.make_weights(H, I, E, 0, dev)
    state = moe.prepare(weights, n_experts=E, top_k=k, max_tokens=max_tokens, token_tile=args.token_tile,
                        decode_path=args.decode_path)
    del weights
    torch.cuda.empty_cache()
    sweeper = moe.L2Sweep(dev)    # 256 MiB > 126 MB of L2
    flush_fn = sweeper.buf.zero_ if args.flush == "write" else sweeper.sweep
    if args.profile_only:
        for i in range(max(args.warmup, 1) + args.steps):
            data, _ = inputs.make_inputs(spec["shape"], T, i % POOL, dev)
            flush_fn()
            moe.kernel_fn(data, state)
        torch.cuda.synchronize()
        print(json.dumps({"profile_only": spec["name"], "plan": moe.plan(state, T), "status": moe.read_status(state)}))
        return

    head = measure(moe, inputs, state, spec, args.steps, args.warmup, peaks, dev, flush_fn)
    workspace_bytes = state["workspace_bytes"]
    sweep = []
    for w in sweep_specs:
        n = max(5, min(args.steps, 20 if w["T"] > 1024 else 100))
        sweep.append(measure(moe, inputs, state, w, n, min(args.warmup, 5), peaks, dev, flush_fn))
    # the few-token points once more with rotating weight sets instead of the L2 sweep
    rot_targets = [m for m in [head] + sweep if m["tokens"] <= 256]
    if rot_targets and args.weight_sets > 1:
        del state
        torch.cuda.empty_cache()
        rot_tokens = max(m["tokens"] for m in rot_targets)
        states = []
        for r in range(args.weight_sets):
            wr = inputs.make_weights(H, I, E, 100 + r, dev)
            states.append(moe.prepare(wr, n_experts=E, top_k=k, max_tokens=rot_tokens, token_tile=args.token_tile,
                                      decode_path=args.decode_path))
            del wr
        torch.cuda.empty_cache()
        by_name = {w["name"]: w for w in [spec] + sweep_specs}
        for m in rot_targets:
            m["weights_rotated"] = measure_rotating(moe, inputs, states, by_name[m["workload"]],
                                                    max(m["steps"], 200), args.warmup, peaks, dev)
        del states
    cpu_base, _ = cpu_oracle_run(spec, 2, cpu_sample_tokens(spec))

    line = {
        "metric": METRIC, "value": head["value"], "unit": UNIT, "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": head["ms_per_step"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": DTYPE, "data": "synthetic",
        "config": {"workload": spec["name"], "tokens": T, "hidden": H, "inter": I, "experts": E, "top_k": k,
                   "l2": ("flushed before every timed step by " + ("zeroing" if args.flush == "write" else "reading")
                          + " a 256 MiB buffer; CUDA-graph replays")},
        "plan": dict(head["plan"], workspace_bytes=workspace_bytes, build_id=_lib.build_id()),
        "e2e": head["e2e"],
        "gpu_launches": head["gpu_launches_per_step"] * args.steps,
        "roofline": head["roofline"], "step_roofline": head["step_roofline"], "kernel_ms": head["kernel_ms"],
        "weights_rotated": head.get("weights_rotated"),
        "cpu_baseline": cpu_base, "clocks": head["clocks"],
        "sweep": sweep,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------ expert parallel, N GPUs
def run_ep(args, spec, dev):
    """--gpus N > 1: config 4 (H7168 I2048 E256 top-8, T = 4096 per GPU), one rank per GPU."""
    import torch
    import torch.distributed as dist
    import muse_moe_w4a16 as moe
    from muse_moe_w4a16 import _lib, ep, inputs

    world, rank = int(os.environ["WORLD_SIZE"]), int(os.environ["RANK"])
    dist.init_process_group("nccl", device_id=dev)
    s = inputs.SHAPES[spec["shape"]]
    H, I, E, k, T = s["H"], s["I"], s["E"], s["k"], spec["T"]
    per = E // world
    CHECK = max(8, 256 // world)   # tokens per rank checked against the one-GPU step

    def rank_weights(r):
        return inputs.make_weights_random_bytes(H, I, per, 1000 + r, dev)

    def rank_input(r, i):
        return inputs.make_inputs(spec["shape"], T, 17 * r + i, dev)[0]

    # rank 0, alone: the same shape with all experts on one GPU -> reference rows for every rank, and the
    # one-GPU step time of the same per-GPU token count
    single_ms = torch.zeros(1, device=dev)
    ref_rows = torch.zeros((world, CHECK, H), dtype=torch.bfloat16, device=dev)
    if rank == 0:
        parts = [rank_weights(r) for r in range(world)]
        allw = {key: torch.cat([p[key].view(torch.uint8) if p[key].dtype == torch.float8_e4m3fn else p[key] for p in parts])
                for key in parts[0]}
        del parts
        st1 = moe.prepare(allw, n_experts=E, top_k=k, max_tokens=T)
        del allw
        torch.cuda.empty_cache()
        for r in range(world):
            d = rank_input(r, 0)
            ref_rows[r] = moe.kernel_fn({"hidden_states": d["hidden_states"][:CHECK].contiguous(),
                                         "router_logits": d["router_logits"][:CHECK].contiguous()}, st1)
        d = rank_input(0, 0)
        for _ in range(3):
            moe.kernel_fn(d, st1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for i in range(5):
            moe.kernel_fn(d, st1)
        e1.record()
        torch.cuda.synchronize()
        single_ms[0] = e0.elapsed_time(e1) / 5
        if moe.read_status(st1) != 0:
            raise RuntimeError("device status word is non-zero in the one-GPU reference step")
        del st1, d
        torch.cuda.empty_cache()
    dist.broadcast(single_ms, 0)
    dist.broadcast(ref_rows, 0)

    chunks = None
    if args.ep_chunks:
        chunks = [int(v) for v in args.ep_chunks.split(",")] if "," in args.ep_chunks else int(args.ep_chunks)
    mod = ep.EPModule(rank_weights(rank), rank, world, E, k, T, chunks=chunks)
    torch.cuda.empty_cache()
    pool = [rank_input(rank, i) for i in range(4)]
    host_pool = [{"hidden_states": d["hidden_states"].cpu().pin_memory(),
                  "router_logits": d["router_logits"].cpu().pin_memory()} for d in pool]

    # parity: this rank's first CHECK tokens of input 0 through the expert-parallel step
    got = mod.kernel_fn(pool[0])[:CHECK].float()
    want = ref_rows[rank].float()
    rel = ((got - want).abs().max() / want.abs().max().clamp_min(1e-30)).reshape(1)
    dist.all_reduce(rel, op=dist.ReduceOp.MAX)
    ep_parity = float(rel.item())

    sampler = ClockSampler(dev.index).start()

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
    timeline = None
    if args.ep_timeline and mod.exchange is not None:
        # where a step's time goes: CUDA events on the main stream of every rank (ms after the step's start;
        # median of 5 steps), reduced to the slowest rank per mark
        rows = []
        for i in range(7):
            mod.exchange.marks = []
            dist.barrier()
            mod.kernel_fn(pool[i % len(pool)])
            torch.cuda.synchronize()
            if i >= 2:
                m0 = mod.exchange.marks[0][1]
                rows.append([m0.elapsed_time(ev) for _, ev in mod.exchange.marks])
        labels = [lab for lab, _ in mod.exchange.marks]
        mod.exchange.marks = None
        med = torch.tensor(rows, device=dev).median(0).values
        worst, best = med.clone(), med.clone()
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        dist.all_reduce(best, op=dist.ReduceOp.MIN)
        timeline = {lab: {"max_ms": float(a), "min_ms": float(b)} for lab, a, b in zip(labels, worst.tolist(), best.tolist())}
    status = torch.tensor([moe.read_status(mod.state)], device=dev)
    dist.all_reduce(status, op=dist.ReduceOp.MAX)
    if int(status.item()) != 0:
        raise RuntimeError("device status word is non-zero on some rank")
    if ep_parity > 1e-2:
        raise RuntimeError(f"expert-parallel output differs from the one-GPU step: max-abs-rel {ep_parity:.3e}")
    if rank == 0:
        peaks = load_peaks()
        flops = inputs.algorithmic_flops(H, I, T * k * world) * args.steps
        step_ms = ms / args.steps
        line = {
            "metric": METRIC, "value": T * world * args.steps / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": step_ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": DTYPE,
            "data": "synthetic",
            "config": {"workload": spec["name"], "tokens_per_gpu": T, "hidden": H, "inter": I, "experts": E,
                       "top_k": k, "parallelism": f"ep{world}",
                       "l2": "inputs and weights exceed L2 (792 MB of weights per rank at 8 ranks)",
                       "dispatch": f"{mod.transport}, source ranks in chunks of {mod.sizes}", "build_id": _lib.build_id()},
            "e2e": {"value": T * world * args.steps / (ms_e2e * 1e-3), "unit": UNIT,
                    "h2d_bytes_per_step": (T * H * 2 + T * E * 4) * world, "d2h_bytes_per_step": T * H * 2 * world,
                    "ms_per_step": ms_e2e / args.steps},
            # per rank and step: top-k, the final rank-order sum, and per chunk the sort (three launches from
            # 16384 entries on), the F16 row copy, two GEMMs and the combine
            "gpu_launches": (2 + sum(7 if m * T * k >= 16384 else 5 for m in mod.sizes)) * args.steps * world,
            "ep_parity_max_rel": ep_parity, "ep_parity_tokens_per_rank": CHECK,
            "single_gpu_same_shape_ms": float(single_ms.item()),
            "scaling_efficiency": float(single_ms.item()) / step_ms,
            "roofline": {"bound": "tensor", "achieved": flops / world / (ms * 1e-3) / 1e12,
                         "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
                         "frac": flops / world / (ms * 1e-3) / 1e12 / peaks["bf16_tflops_sustained"],
                         "frac_of_burst_peak": flops / world / (ms * 1e-3) / 1e12 / peaks["bf16_tflops"], "traffic": None,
                         "kernel": "whole EP step per GPU (expert kernels + exchange)",
                         "peak_source": peaks["source"] + " (sustained; burst beside it)"},
            "cpu_baseline": None,
            "clocks": clocks,
        }
        if timeline is not None:
            line["ep_timeline_ms"] = timeline
        print(json.dumps(line), flush=True)
    dist.barrier()
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--workload", default="auto")
    ap.add_argument("--no-sweep", action="store_true", help="one GPU, default workload: leave out the other points of the metric")
    ap.add_argument("--experts", type=int, default=0, help="resident experts (smaller case for profiler captures)")
    ap.add_argument("--ep-chunks", default="", help="expert-parallel runs: number of equal chunks of source ranks, or their sizes "
                                                    "as a comma list (own rank first), e.g. 1,3,3,1; empty = default")
    ap.add_argument("--ep-timeline", action="store_true", help="expert-parallel runs: add per-chunk event times of a step to the line")
    ap.add_argument("--token-tile", type=int, default=0, help="force the token tile of the GEMM kernels: 16/32/64/128")
    ap.add_argument("--decode-path", type=int, default=0, help="few tokens: 0 auto, 1 chain of launches, 2 three launches, 3 one launch")
    ap.add_argument("--weight-sets", type=int, default=6,
                    help="weight sets of the rotating-weights timing of the few-token points (0 or 1: leave it out)")
    ap.add_argument("--flush", default="read", choices=["read", "write"], help="how L2 is flushed before a timed step")
    ap.add_argument("--profile-only", action="store_true", help="run warmup+steps eager steps and exit (for ncu)")
    args = ap.parse_args()
    spec = workload_spec(args.workload, args.gpus)
    # Standard output carries the one JSON line and nothing else: libraries that write to file descriptor 1
    # themselves (NCCL prints its version there when the first communicator comes up) go to standard error.
    sys.stdout.flush()
    line_fd = os.dup(1)
    os.dup2(2, 1)
    sys.stdout = os.fdopen(line_fd, "w")
    if args.impl == "reference":
        run_reference(args, spec)
    else:
        run_gpu(args, spec)
    sys.stdout.flush()


if __name__ == "__main__":
    main()
