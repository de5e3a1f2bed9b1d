"""Expert parallelism for the routed-expert step.

Rank r of n owns experts [r*E/n, (r+1)*E/n) (the reference's `local_start / local_count`
convention, muse_moe_w4a16/py/00_moe_w4a16.py:108-109; the reference itself only filters ids
and leaves the exchange to its caller, muse_moe_w4a16/cuda/moe.cu:347-350). Every rank holds
T tokens. One step:
  1. routing on the local tokens (global ids, weights);
  2. dispatch: every rank receives every rank's token rows with their ids/weights rows. Sending
     a token only to the ranks it routes to would need per-destination sizes on the host or
     padded buffers of the same T rows per pair; with top-8 of 8 ranks two thirds of the pairs
     are used anyway, so rows travel whole and the step has no host synchronisation;
  3. the local expert step in the reference's filter mode: ids outside this rank's range are
     skipped by the sort, giving one partial row per received token (zero without a route here);
  4. combine: the partial rows return to the token's home rank, which sums them in rank order in
     FP32 (deterministic), reading only the ranks the token routed to.

Two transports:
  * "collective": all_gather + all_to_all_single of torch.distributed (gloo in the CPU tests,
    NCCL on GPUs), one chunk, nothing overlapped;
  * "symm" (GPUs of one NVLink domain): buffers in symmetric memory, rows pulled from the peers
    by the copy engines (plain device-to-device copies, no SM), cross-rank ordering by 32-bit
    flags written and awaited with stream memory operations. The n source ranks are processed
    in chunks, own rank first, so the expert kernels of one chunk run while the copy engines
    fetch the next chunk and return the previous one. Remote data always lands in this rank's
    own memory before a kernel reads it.
"""
import ctypes

import torch
import torch.distributed as dist


def wait_deadline(event, seconds, what):
    """Host-side deadline for a stream that may be blocked on a peer's flag: polls event.query() and
    raises TimeoutError after `seconds`. A flag wait is a stream operation that the device cannot
    bound; a peer that died would block this rank's stream until the launcher ends the job, so callers
    that need to notice sooner (at the price of one host synchronisation per step) poll here."""
    import time

    t0 = time.time()
    while not event.query():
        if time.time() - t0 > seconds:
            raise TimeoutError(f"expert-parallel exchange: {what} did not complete within {seconds} s (a peer is not answering)")
        time.sleep(0.0005)


def chunk_sizes(world, chunks=None):
    """How the `world` source ranks (slot 0 = this rank's own tokens, slot j = rank + j) are grouped into
    chunks that are processed one after the other. chunks: None (default), a number of equal chunks,
    or the sizes themselves. The default starts with the rank's own tokens alone (they need no transfer,
    so nothing is waited for at the head of the step), ends with a single source rank (so that only
    one rank's partial rows are still on their way back when the expert kernels have finished) and
    takes the ranks in between two at a time (measured on 8 B200s, 4096 tokens per GPU:
    [1, 2, 2, 2, 1] 3.87 ms, [1, 3, 3, 1] 3.99 ms, [2, 2, 2, 2] 4.12 ms a step)."""
    if chunks is None:
        if world <= 2:
            return [world]
        if world == 3:
            return [1, 2]
        mid = world - 2
        return [1] + [2] * (mid // 2) + ([1] if mid % 2 else []) + [1]
    if isinstance(chunks, int):
        if chunks < 1 or world % chunks != 0:
            raise ValueError("the number of chunks must divide the number of ranks")
        return [world // chunks] * chunks
    sizes = [int(v) for v in chunks]
    if sum(sizes) != world or min(sizes) < 1:
        raise ValueError("chunk sizes must be positive and add up to the number of ranks")
    return sizes


def owner_rank(ids, experts_per_rank):
    return torch.div(ids, experts_per_rank, rounding_mode="floor")


def route_mask(ids, n_ranks, experts_per_rank):
    """ids [T, k] (global, negative = no route) -> bool [n, T]: token t has a route on rank d."""
    dest = owner_rank(ids.long(), experts_per_rank)
    ranks = torch.arange(n_ranks, device=ids.device).view(n_ranks, 1, 1)
    return ((dest.unsqueeze(0) == ranks) & (ids.unsqueeze(0) >= 0)).any(-1)


def combine_partials(back, ids, experts_per_rank, self_rank=-1, self_rows=None):
    """out[t] = bf16(sum over ranks d, in rank order, of rank d's partial row of token t, taken only
    where the token routes to d), FP32 accumulation. back bf16 [n, T, H] in rank order; self_rows
    replaces back[self_rank] when given. On CUDA tensors this is one library kernel
    (msk_ep_combine); the torch loop is the same arithmetic for the CPU ranks of the tests."""
    n, T, H = back.shape
    if back.is_cuda:
        from . import _lib

        out = torch.empty((T, H), dtype=torch.bfloat16, device=back.device)
        ids32 = ids.to(torch.int32).contiguous()
        _lib.check(_lib.load().msk_ep_combine(_lib.ptr(back), _lib.ptr(self_rows), self_rank, _lib.ptr(ids32),
                                              ids32.shape[1], experts_per_rank, _lib.ptr(out), n, T, H,
                                              ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)),
                   "msk_ep_combine")
        return out
    mask = route_mask(ids, n, experts_per_rank)
    out = torch.zeros((T, H), dtype=torch.float32, device=back.device)
    for d in range(n):                                                       # rank order, FP32
        rows = self_rows if (d == self_rank and self_rows is not None) else back[d]
        out += torch.where(mask[d].unsqueeze(-1), rows.float(), torch.zeros((), dtype=torch.float32))
    return out.to(torch.bfloat16)


def _all_gather(t, n, group):
    out = torch.empty((n,) + tuple(t.shape), dtype=t.dtype, device=t.device)
    if t.is_cuda:
        dist.all_gather_into_tensor(out, t.contiguous(), group=group)
    else:                                   # gloo: per-rank views, moved as bytes
        dist.all_gather([out[d].view(torch.uint8) for d in range(n)], t.contiguous().view(torch.uint8), group=group)
    return out


def ep_step(x, ids, weights, expert_fn, experts_per_rank, group=None):
    """The step over torch.distributed collectives. x bf16 [T, H], ids int [T, k] (global ids),
    weights fp32 [T, k]. expert_fn(rows bf16 [n*T, H], ids int32 [n*T, k], weights fp32 [n*T, k])
    -> partial bf16 [n*T, H] computes this rank's experts (ids outside its range or negative are
    skipped). Returns out bf16 [T, H]."""
    n = dist.get_world_size(group)
    T, H = x.shape
    k = ids.shape[1]
    ids32 = ids.to(torch.int32)
    rows = _all_gather(x, n, group).view(n * T, H)
    rids = _all_gather(ids32, n, group).view(n * T, k)
    rw = _all_gather(weights.float(), n, group).view(n * T, k)
    partial = expert_fn(rows, rids, rw)                                      # [n*T, H] bf16
    back = torch.empty((n, T, H), dtype=partial.dtype, device=partial.device)
    dist.all_to_all_single(back, partial.view(n, T, H).contiguous(), group=group)   # back[d]: rank d's rows for my tokens
    return combine_partials(back, ids32, experts_per_rank)


class SymmExchange:
    """Buffers, flags and the copy stream of the "symm" transport for one rank.

    Symmetric buffers (same shape on every rank, peers mapped into this address space), two
    copies each, used by steps of alternating parity so a rank never overwrites rows a slower
    peer may still be pulling:
      gx/gids/gtw [2, n, T, ...]  slot 0: this rank's rows (what the peers pull); slot j: the rows
                                  of rank (rank + j) % n, pulled by this rank;
      part        [2, n, T, H]    slot j: this rank's partial rows for the tokens of rank
                                  (rank + j) % n (what that rank pulls back);
      flags       int32 [4 n]     word 2 p + b: rank p's inputs of a parity-b step are in place;
                                  word 2 n + 2 q + b: rank q has written its partial rows for this
                                  rank's tokens. Values are step numbers, compared with >=.
    Why two copies are enough: a rank reaches step e + 2 only after it pulled every peer's
    partial rows of step e + 1, and a peer produces those after its own pulls of step e + 1,
    which its copy stream runs after its pulls of step e.
    """

    def __init__(self, rank, world, tokens, hidden, top_k, chunks, device, group=None):
        import torch.distributed._symmetric_memory as symm

        from . import _lib

        self.rank, self.n, self.T, self.H, self.k = rank, world, tokens, hidden, top_k
        self.sizes = chunk_sizes(world, chunks)
        self.chunks = len(self.sizes)
        self.bounds = [sum(self.sizes[:i]) for i in range(self.chunks + 1)]   # chunk c = slots [bounds[c], bounds[c+1])
        self.lib = _lib.load()
        g = group if group is not None else dist.group.WORLD

        def alloc(shape, dtype):
            t = symm.empty(shape, dtype=dtype, device=device)
            h = symm.rendezvous(t, g)
            peers = [h.get_buffer(p, shape, dtype) for p in range(world)]
            return t, h, peers

        n, T, H, k = world, tokens, hidden, top_k
        self.gx, _, self.peer_gx = alloc((2, n, T, H), torch.bfloat16)
        self.gids, _, self.peer_gids = alloc((2, n, T, k), torch.int32)
        self.gtw, _, self.peer_gtw = alloc((2, n, T, k), torch.float32)
        self.part, _, self.peer_part = alloc((2, n, T, H), torch.bfloat16)
        self.flags, hf, _ = alloc((4 * n,), torch.int32)
        self.flags.zero_()
        self.flag_base = [int(p) for p in hf.buffer_ptrs]
        self.back = torch.empty((n, T, H), dtype=torch.bfloat16, device=device)
        self.comm = torch.cuda.Stream(device)
        self.epoch = 0
        self.marks = None      # set to a list to have step() record (label, CUDA event) pairs on the main stream
        torch.cuda.synchronize(device)
        dist.barrier(group)                      # every rank's flags are zero before anyone writes

    def _write(self, peer, word, value, stream):
        from . import _lib

        _lib.check(self.lib.msk_ep_flag_write(ctypes.c_void_p(self.flag_base[peer] + 4 * word), value,
                                              ctypes.c_void_p(stream.cuda_stream)), "msk_ep_flag_write")

    def _wait(self, word, value, stream):
        from . import _lib

        _lib.check(self.lib.msk_ep_flag_wait(ctypes.c_void_p(self.flag_base[self.rank] + 4 * word), value,
                                             ctypes.c_void_p(stream.cuda_stream)), "msk_ep_flag_wait")

    def step(self, x, ids, tw, expert_fn, experts_per_rank, deadline_s=None):
        """expert_fn(rows, ids, weights, out) as in ep_step, writing its partial rows into `out`.
        deadline_s: when given, the host waits (polling, wait_deadline) until the last pull of the step has
        completed and raises TimeoutError if a peer does not answer in time; None keeps the step free of
        host synchronisation."""
        n, r, T, H, k = self.n, self.rank, self.T, self.H, self.k
        bounds = self.bounds
        self.epoch += 1
        e, b = self.epoch, self.epoch & 1
        gx, gids, gtw, part = self.gx[b], self.gids[b], self.gtw[b], self.part[b]
        s0, s1 = torch.cuda.current_stream(), self.comm
        def mark(label):
            if self.marks is not None:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record(s0)
                self.marks.append((label, ev))

        mark("start")
        gx[0].copy_(x)
        gids[0].copy_(ids)
        gtw[0].copy_(tw)
        ev_in = torch.cuda.Event()
        ev_in.record(s0)
        for j in range(1, n):
            self._write((r + j) % n, 2 * r + b, e, s0)
        def run_chunk(c):
            mark(f"chunk{c}_rows_in")
            sl, m = slice(bounds[c], bounds[c + 1]), self.sizes[c]
            expert_fn(gx[sl].view(m * T, H), gids[sl].view(m * T, k), gtw[sl].view(m * T, k), part[sl].view(m * T, H))
            mark(f"chunk{c}_experts_done")
            for j in range(max(bounds[c], 1), bounds[c + 1]):
                self._write((r + j) % n, 2 * n + 2 * r + b, e, s0)

        # A first chunk that holds this rank's own rows only needs no transfer: its launches are issued
        # before the host spends its time on the copy stream's calls below (some forty of them; issued
        # first they kept the main stream idle for a quarter of a millisecond at the head of the step)
        own_first = self.sizes[0] == 1
        if own_first:
            run_chunk(0)
        # copy stream: pull the other ranks' rows, nearest rank first
        s1.wait_event(ev_in)
        ready = {}
        with torch.cuda.stream(s1):
            for j in range(1, n):
                p = (r + j) % n
                self._wait(2 * p + b, e, s1)
                gx[j].copy_(self.peer_gx[p][b, 0], non_blocking=True)
                gids[j].copy_(self.peer_gids[p][b, 0], non_blocking=True)
                gtw[j].copy_(self.peer_gtw[p][b, 0], non_blocking=True)
                if j + 1 in bounds:                      # the last slot of a chunk has been issued
                    c = bounds.index(j + 1) - 1
                    ready[c] = torch.cuda.Event()
                    ready[c].record(s1)
        # main stream: the local expert step chunk by chunk
        for c in range(1 if own_first else 0, self.chunks):
            if c in ready:
                s0.wait_event(ready[c])
            run_chunk(c)
        # copy stream: pull this rank's partial rows back, in the order the peers finish them
        with torch.cuda.stream(s1):
            for j in range(1, n):
                q = (r - j) % n
                self._wait(2 * n + 2 * q + b, e, s1)
                self.back[q].copy_(self.peer_part[q][b, j], non_blocking=True)
            ev_back = torch.cuda.Event()
            ev_back.record(s1)
        if deadline_s is not None:
            wait_deadline(ev_back, deadline_s, f"step {e} on rank {r}")
        s0.wait_event(ev_back)
        mark("partials_back")
        out = combine_partials(self.back, gids[0], experts_per_rank, self_rank=r, self_rows=part[0])
        mark("combined")
        return out


class EPModule:
    """prepare/kernel_fn for one rank of an expert-parallel group."""

    def __init__(self, local_weights, rank, world, n_experts, top_k, tokens_per_rank, group=None, transport="symm",
                 chunks=None, deadline_s=None, **prep):
        import muse_moe_w4a16 as moe

        self.moe, self.rank, self.world, self.group = moe, rank, world, group
        self.n_experts, self.top_k, self.per_rank = n_experts, top_k, n_experts // world
        self.transport = transport
        self.deadline_s = deadline_s
        if transport == "symm":
            sizes = chunk_sizes(world, chunks)
            self.sizes = sizes
            self.chunks, rows = len(sizes), max(sizes) * tokens_per_rank
        elif transport == "collective":
            self.sizes = [world]
            self.chunks, rows = 1, world * tokens_per_rank
        else:
            raise ValueError("transport must be 'symm' or 'collective'")
        self.state = moe.prepare(local_weights, local_start=rank * self.per_rank, n_experts=n_experts, top_k=top_k,
                                 max_tokens=rows, **prep)
        self.exchange = None
        if transport == "symm":
            dev = self.state["packed13"].device
            self.exchange = SymmExchange(rank, world, tokens_per_rank, self.state["cfg"].hidden, top_k, chunks, dev, group)

    def _experts(self, rows, ids, w, out=None):
        return self.moe.kernel_fn({"hidden_states": rows, "topk_ids": ids, "topk_weights": w}, self.state, out=out)

    def route(self, logits):
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
        if self.exchange is not None:
            return self.exchange.step(x, ids, tw, self._experts, self.per_rank, deadline_s=self.deadline_s)
        return ep_step(x, ids, tw, self._experts, self.per_rank, self.group)
