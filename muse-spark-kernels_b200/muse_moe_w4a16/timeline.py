"""Per-CTA timeline of one MoE step from the kernels' own %globaltimer stamps.

    python -m muse_moe_w4a16.timeline <shape> <tokens> [key=value ...] [--flush read|write|none] [--replays N] [--pool N]

<shape> names an entry of inputs.SHAPES (decode, sweep, prefill ...); key=value pairs go to prepare()
(decode_path=2, flat_shares=1, num_ctas=128 ...). The step is captured in CUDA graphs over a pool of
inputs and replayed with the L2 swept before each replay, as the benchmark runs it; prepare(trace=1)
makes every CTA of the GEMM launches store a stamp where each stage of its pipeline first (or last)
happened. Printed: for every stamp the minimum, median and maximum over the CTAs that reached it, in
microseconds after the first CTA of the first GEMM launch started, each the median over the replays.
"""
import argparse

import numpy as np
import torch

from . import L2Sweep, inputs, kernel_fn, plan, prepare, read_status, trace_stamps

# stamp slot of every name, in the order a CTA passes them (gemm.cuh, enum TraceSlot)
STAMPS = (("START", 0), ("CONVERTED", 12), ("TOPK", 13), ("ROUTED", 10), ("SETUP", 1), ("FIRST_BULK", 2),
          ("FIRST_RAW", 3), ("FIRST_AFULL", 4), ("FIRST_MMA", 5), ("FIRST_DFULL", 6), ("FIRST_EPI_DONE", 7),
          ("LAST_DFULL", 8), ("FOLD_END", 11), ("END", 9))
LAUNCHES = ("gate/up GEMM (or the one-launch kernel)", "down GEMM")


def collect(shape, tokens, replays=8, flush="read", pool_size=4, **prepare_kw):
    """Returns (state, median step us, {(launch, stamp): (min, median, max, n_ctas)})."""
    dev = torch.device("cuda", 0)
    s = inputs.SHAPES[shape]
    weights = inputs.make_weights_random_bytes(s["H"], s["I"], s["E"], 0, dev)
    state = prepare(weights, n_experts=s["E"], top_k=s["k"], max_tokens=tokens, trace=1, **prepare_kw)
    sweep = L2Sweep(dev)
    flush_l2 = {"write": sweep.buf.zero_, "read": sweep.sweep, "none": lambda: None}[flush]
    pool = [inputs.make_inputs(shape, tokens, i, dev)[0] for i in range(pool_size)]
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for d in pool:
            kernel_fn(d, state)
    torch.cuda.current_stream().wait_stream(side)
    graphs = []
    for d in pool:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            kernel_fn(d, state)
        graphs.append(g)
    for i in range(50):
        flush_l2()
        graphs[i % pool_size].replay()
    torch.cuda.synchronize()
    grid = plan(state, tokens)[3]
    acc, steps = {}, []
    for rep in range(replays):
        flush_l2()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graphs[rep % pool_size].replay()
        e1.record()
        torch.cuda.synchronize()
        steps.append(e0.elapsed_time(e1) * 1e3)
        stamps = trace_stamps(state)[0].cpu().numpy()
        starts = stamps[0, :grid, 0]
        t0 = starts[starts > 0].min()
        for launch in range(2):
            t = stamps[launch, :grid, :].astype(np.float64)
            for name, col in STAMPS:
                reached = t[:, col] > t0 - 1e9      # a stamp of this replay, not a stale or empty word
                if reached.any():
                    r = (t[reached, col] - t0) / 1e3
                    acc.setdefault((launch, name), []).append((r.min(), np.median(r), r.max(), reached.sum()))
    table = {k: tuple(np.median(np.array(v), axis=0)) for k, v in acc.items()}
    return state, float(np.median(steps)), table


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("shape")
    ap.add_argument("tokens", type=int)
    ap.add_argument("prepare_kw", nargs="*", help="key=value integers passed to prepare()")
    ap.add_argument("--flush", choices=("read", "write", "none"), default="read",
                    help="none: no sweep between replays (code and part of the weights stay in L2)")
    ap.add_argument("--replays", type=int, default=8)
    ap.add_argument("--pool", type=int, default=4,
                    help="distinct inputs cycled through (1 with --flush none: the touched weights stay in L2)")
    a = ap.parse_args()
    kw = {k: int(v) for k, v in (kv.split("=") for kv in a.prepare_kw)}
    state, step_us, table = collect(a.shape, a.tokens, a.replays, a.flush, a.pool, **kw)
    print(f"# {a.shape} T={a.tokens} plan (tile, path, flat, grid) = {plan(state, a.tokens)}")
    print(f"step (event-timed graph replay, L2 sweep before it: {a.flush}): median {step_us:.1f} us")
    print(f"us after the first CTA of the first GEMM launch started; per stamp min / median / max over CTAs "
          f"(median over {a.replays} replays), CTAs that reached it")
    for launch, title in enumerate(LAUNCHES):
        rows = [(n, table[(launch, n)]) for n, _ in STAMPS if (launch, n) in table]
        if not rows:
            continue
        print(f"## {title}")
        for n, (lo, med, hi, cnt) in rows:
            print(f"  {n:15s} {lo:7.2f} / {med:7.2f} / {hi:7.2f}   ({int(cnt)} CTAs)")
    print("status", read_status(state))


if __name__ == "__main__":
    main()
