"""muse_moe_w4a16 for B200: the reference module's two entry points over libmsk_moe.so.

    state = prepare(weights)            # once; may synchronise; lossless repack only
    out   = kernel_fn(data, state)      # timed path; no host sync; CUDA-graph capturable

`weights` and `data` are the reference's `Weights` / `Inputs` dicts
(muse_moe_w4a16/py/00_moe_w4a16.py:72-97; prepare: py/02_prepare.py:2, kernel_fn:
py/03_kernel_fn.py:18-45). Extensions, all optional:
  weights["router"]       fp32 [E, H]   -> kernel_fn computes logits = x @ router.T in FP32
  weights["route_bias"]   fp32 [E]      -> selection bias of the sigmoid routing mode
  data["router_logits"]   fp32 [T, E]   -> kernel_fn runs top-k itself (ids/weights not needed)
  post_norm_w may be absent             -> plain weighted combine, no post-expert RMS norm
  pre_norm_w (bf16 [H]) may be present  -> the layer callers' pre-expert RMS norm is applied to x first
There is no CPU path: tensors must be CUDA tensors and the native library must load.
"""
import ctypes

import torch

from . import _lib
from ._lib import ROUTE_SIGMOID_BIAS, ROUTE_SOFTMAX_TOPK, MskMoeCfg

__all__ = ["prepare", "kernel_fn", "export_weights", "read_status", "reinit_workspace", "state_dict", "load_state_dict",
           "workspace_views", "attrs", "GraphedStep", "HostMappedStep"]

_MODES = {"softmax_topk": ROUTE_SOFTMAX_TOPK, "sigmoid_bias": ROUTE_SIGMOID_BIAS}


def _u8(t):
    # the decode layer hands the codes over with whatever 1-byte dtype the checkpoint used
    # (muse_decode_layer/py/03_layer_helpers.py:68), so reinterpret instead of converting
    return t.contiguous().view(torch.uint8)


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def prepare(weights, *, local_start=0, n_experts=None, top_k=8, max_tokens=8192, routing_mode="softmax_topk",
            route_scale=0.1767766952966369, post_norm_eps=1e-8, num_ctas=0, decode_path=0, no_pdl=0, token_tile=0,
            trace=0, stop_after=0, pre_norm_eps=1e-5, flat_shares=0):
    """Repack the NVFP4 weights into the tile layout the GEMM kernel streams (bit and byte
    permutations only, never requantised) and allocate the workspace. Returns `state`."""
    w13 = _u8(weights["w13"])
    if not w13.is_cuda:
        raise RuntimeError("muse_moe_w4a16.prepare: weights must be CUDA tensors (there is no CPU path)")
    lib = _lib.load()
    dev = w13.device
    n_local, two_i, half_h = w13.shape
    I, H = two_i // 2, half_h * 2
    w13_sf, w2, w2_sf = _u8(weights["w13_sf"]), _u8(weights["w2"]), _u8(weights["w2_sf"])
    if tuple(w2.shape) != (n_local, H, I // 2) or tuple(w13_sf.shape) != (n_local, 2 * I, H // 16) \
            or tuple(w2_sf.shape) != (n_local, H, I // 16):
        raise RuntimeError("muse_moe_w4a16.prepare: inconsistent weight shapes")
    if weights["w13_gs"].dtype != torch.float32 or weights["w2_gs"].dtype != torch.float32:
        raise RuntimeError("muse_moe_w4a16.prepare: global scales must be float32")
    cfg = MskMoeCfg(hidden=H, inter=I, n_experts=n_experts or n_local, local_start=local_start,
                    local_count=n_local, top_k=top_k, routing_mode=_MODES[routing_mode], route_scale=route_scale,
                    post_norm_eps=post_norm_eps, num_ctas=num_ctas, decode_path=decode_path, no_pdl=no_pdl,
                    token_tile=token_tile, max_tokens=max_tokens, trace=trace, stop_after=stop_after,
                    flat_shares=flat_shares)
    b13, b2 = ctypes.c_size_t(), ctypes.c_size_t()
    _lib.check(lib.msk_moe_packed_bytes(ctypes.byref(cfg), ctypes.byref(b13), ctypes.byref(b2)), "msk_moe_packed_bytes")
    with torch.cuda.device(dev):
        packed13 = torch.empty(b13.value, dtype=torch.uint8, device=dev)
        packed2 = torch.empty(b2.value, dtype=torch.uint8, device=dev)
        _lib.check(lib.msk_moe_repack(ctypes.byref(cfg), _lib.ptr(w13), _lib.ptr(w13_sf), _lib.ptr(w2), _lib.ptr(w2_sf),
                                      _lib.ptr(packed13), _lib.ptr(packed2), _stream()), "msk_moe_repack")
    prw = weights.get("pre_norm_w")
    if prw is not None and (prw.dtype != torch.bfloat16 or prw.numel() != 2 * weights["w13"].shape[2]):
        raise RuntimeError("muse_moe_w4a16.prepare: pre_norm_w must be bfloat16 [hidden]")
    pnw = weights.get("post_norm_w")
    if pnw is not None and pnw.dtype != torch.bfloat16:
        raise RuntimeError("muse_moe_w4a16.prepare: post_norm_w must stay bfloat16")
    return _make_state(cfg, packed13, packed2, weights["w13_gs"], weights["w2_gs"], pnw, prw, pre_norm_eps,
                       weights.get("router"), weights.get("route_bias"))


ROUTER_GEMM_MIN_TOKENS = 16   # from here on the router logits come from the tensor-core GEMM


def split_router(router):
    """FP32 router weight [E, H] -> bf16 [2E, H] = [hi; lo] with hi = bf16(w), lo = bf16(w - hi): the
    pair whose sum the reference's layers feed to their BF16 GEMM
    (muse_decode_layer/py/05_tune.py:279-286, muse_prefill_layer/py/00_layer.py:369-374)."""
    w = router.float()
    hi = w.to(torch.bfloat16)
    lo = (w - hi.float()).to(torch.bfloat16)
    return torch.cat([hi, lo], 0).contiguous()


def _make_state(cfg, packed13, packed2, gs13, gs2, post_norm_w, pre_norm_w, pre_norm_eps, router, route_bias):
    """The state dict around already packed weights: allocates and initialises the workspace."""
    lib = _lib.load()
    dev = packed13.device
    with torch.cuda.device(dev):
        wsb = ctypes.c_size_t()
        _lib.check(lib.msk_moe_workspace_bytes(ctypes.byref(cfg), ctypes.byref(wsb)), "msk_moe_workspace_bytes")
        workspace = torch.empty(wsb.value, dtype=torch.uint8, device=dev)
        _lib.check(lib.msk_moe_workspace_init(ctypes.byref(cfg), _lib.ptr(workspace), wsb.value, _stream()),
                   "msk_moe_workspace_init")
        torch.cuda.synchronize(dev)
    return {
        "cfg": cfg, "lib": _lib.LibHandle(), "lo": cfg.local_start, "cnt": cfg.local_count,
        "packed13": packed13, "packed2": packed2,
        "gs13": gs13.contiguous(), "gs2": gs2.contiguous(),
        "post_norm_w": None if post_norm_w is None else post_norm_w.contiguous(),
        "pre_norm_w": None if pre_norm_w is None else pre_norm_w.contiguous(),
        "pre_norm_eps": float(pre_norm_eps),
        "router": None if router is None else router.float().contiguous(),
        "router_hilo": None if router is None else split_router(router),
        "route_bias": None if route_bias is None else route_bias.float().contiguous(),
        "workspace": workspace, "workspace_bytes": wsb.value,
    }


_SD_TENSORS = ("packed13", "packed2", "gs13", "gs2", "post_norm_w", "pre_norm_w", "router", "route_bias")


def state_dict(state):
    """What a checkpoint needs to rebuild `state` without the original weights and without the repack:
    the packed weight tiles, the scales and norm weights, and the configuration as plain numbers. The
    workspace is scratch and is not part of it. (The reference keeps no such state: its prepare() is
    re-run from the weights every time, muse_moe_w4a16/py/02_prepare.py:2-81.)"""
    cfg = state["cfg"]
    sd = {k: state[k] for k in _SD_TENSORS if state.get(k) is not None}
    sd["config"] = {name: getattr(cfg, name) for name, _ in MskMoeCfg._fields_}
    sd["pre_norm_eps"] = state["pre_norm_eps"]
    return sd


def load_state_dict(sd, device=None):
    """Inverse of state_dict: a ready state on `device` (default: where the tensors are). No repack runs;
    the packed tiles are taken as they are, so kernel_fn gives the same bits as on the state they came from."""
    lib = _lib.load()
    cfg = MskMoeCfg(**sd["config"])
    t = {k: (sd[k] if device is None else sd[k].to(device)) for k in _SD_TENSORS if sd.get(k) is not None}
    if not t["packed13"].is_cuda:
        raise RuntimeError("muse_moe_w4a16.load_state_dict: tensors must be CUDA tensors (there is no CPU path)")
    b13, b2 = ctypes.c_size_t(), ctypes.c_size_t()
    _lib.check(lib.msk_moe_packed_bytes(ctypes.byref(cfg), ctypes.byref(b13), ctypes.byref(b2)), "msk_moe_packed_bytes")
    if t["packed13"].numel() != b13.value or t["packed2"].numel() != b2.value:
        raise RuntimeError("muse_moe_w4a16.load_state_dict: packed weights do not match the configuration")
    return _make_state(cfg, t["packed13"].contiguous(), t["packed2"].contiguous(), t["gs13"], t["gs2"],
                       t.get("post_norm_w"), t.get("pre_norm_w"), sd.get("pre_norm_eps", 1e-5), t.get("router"),
                       t.get("route_bias"))


def reinit_workspace(state):
    """Puts the control words of the workspace back to their initial state (status word, tickets, grid
    and tile counters). Call it when read_status() returned non-zero before using the state again: a
    kernel that gave up on a bounded wait leaves tickets and counters half-way, and the status word is
    sticky. Synchronises."""
    _lib.check(state["lib"].lib.msk_moe_workspace_init(ctypes.byref(state["cfg"]), _lib.ptr(state["workspace"]),
                                                       state["workspace_bytes"], _stream()), "msk_moe_workspace_init")
    torch.cuda.synchronize(state["workspace"].device)


def _logits(data, state, x, T):
    """Router logits of this call: given, or x @ router^T computed by the library; None when the
    caller supplies ids and weights."""
    cfg, lib = state["cfg"], state["lib"].lib
    if data.get("topk_ids") is not None:
        return None
    logits = data.get("router_logits")
    if logits is None:
        if state["router"] is None:
            raise RuntimeError("muse_moe_w4a16.kernel_fn: need topk_ids/topk_weights, router_logits or weights['router']")
        logits = torch.empty((T, cfg.n_experts), dtype=torch.float32, device=x.device)
        if T >= ROUTER_GEMM_MIN_TOKENS and state.get("router_hilo") is not None and state.get("router_gemm", True):
            # tensor-core GEMM on the BF16 hi + lo pair of the router weight
            _lib.check(lib.msk_moe_router_logits_hilo(ctypes.byref(cfg), _lib.ptr(x), _lib.ptr(state["router_hilo"]),
                                                      _lib.ptr(logits), _lib.ptr(state["workspace"]), T, _stream()),
                       "msk_moe_router_logits_hilo")
        else:   # few tokens: FP32 matvec in a fixed summation order
            _lib.check(lib.msk_moe_router_logits(ctypes.byref(cfg), _lib.ptr(x), _lib.ptr(state["router"]),
                                                 _lib.ptr(logits), T, _stream()), "msk_moe_router_logits")
    return logits.to(torch.float32).contiguous()


def _route(data, state, x, T):
    """ids and weights as separate launches (used by the measuring entry point)."""
    cfg, lib = state["cfg"], state["lib"].lib
    logits = _logits(data, state, x, T)
    if logits is None:
        return data["topk_ids"].to(torch.int32).contiguous(), data["topk_weights"].to(torch.float32).contiguous()
    ids = torch.empty((T, cfg.top_k), dtype=torch.int32, device=x.device)
    tw = torch.empty((T, cfg.top_k), dtype=torch.float32, device=x.device)
    _lib.check(lib.msk_moe_route(ctypes.byref(cfg), _lib.ptr(logits), _lib.ptr(state["route_bias"]), _lib.ptr(ids),
                                 _lib.ptr(tw), T, _stream()), "msk_moe_route")
    return ids, tw


def kernel_fn(data, state, return_routing=False, out=None):
    """One routed-expert step. Fresh bf16 [T, H] output per call (or `out`, a contiguous bf16 [T, H]
    CUDA tensor of the caller); launches only."""
    cfg, lib = state["cfg"], state["lib"].lib
    x = data["hidden_states"].contiguous()
    if not x.is_cuda or x.dtype != torch.bfloat16:
        raise RuntimeError("muse_moe_w4a16.kernel_fn: hidden_states must be a CUDA bfloat16 tensor")
    T = x.shape[0]
    dcfg = data.get("config")
    if dcfg is not None and (dcfg["local_start"] != state["lo"] or dcfg["local_count"] != state["cnt"]):
        raise RuntimeError("muse_moe_w4a16.kernel_fn: config local range differs from the prepared state")
    if out is None:
        out = torch.empty((T, cfg.hidden), dtype=torch.bfloat16, device=x.device)
    elif (not out.is_cuda or out.dtype != torch.bfloat16 or not out.is_contiguous()
          or tuple(out.shape) != (T, cfg.hidden)):
        raise RuntimeError("muse_moe_w4a16.kernel_fn: out must be a contiguous CUDA bfloat16 [T, H] tensor")
    logits = _logits(data, state, x, T)
    if state.get("pre_norm_w") is not None:
        # the layer callers' pre-expert RMS norm, fused into the kernel that copies the token rows
        if logits is None:
            ids = data["topk_ids"].to(torch.int32).contiguous()
            tw = data["topk_weights"].to(torch.float32).contiguous()
        else:
            ids = torch.empty((T, cfg.top_k), dtype=torch.int32, device=x.device)
            tw = torch.empty((T, cfg.top_k), dtype=torch.float32, device=x.device)
        _lib.check(lib.msk_moe_forward_prenorm(ctypes.byref(cfg), _lib.ptr(state["packed13"]), _lib.ptr(state["packed2"]),
                                               _lib.ptr(state["gs13"]), _lib.ptr(state["gs2"]),
                                               _lib.ptr(state["post_norm_w"]), _lib.ptr(state["pre_norm_w"]),
                                               ctypes.c_float(state["pre_norm_eps"]), _lib.ptr(x), _lib.ptr(logits),
                                               _lib.ptr(state["route_bias"]), _lib.ptr(ids), _lib.ptr(tw), _lib.ptr(out),
                                               _lib.ptr(state["workspace"]), state["workspace_bytes"], T, _stream()),
                   "msk_moe_forward_prenorm")
        return (out, ids, tw) if return_routing else out
    if logits is None:
        ids = data["topk_ids"].to(torch.int32).contiguous()
        tw = data["topk_weights"].to(torch.float32).contiguous()
        _lib.check(lib.msk_moe_forward(ctypes.byref(cfg), _lib.ptr(state["packed13"]), _lib.ptr(state["packed2"]),
                                       _lib.ptr(state["gs13"]), _lib.ptr(state["gs2"]), _lib.ptr(state["post_norm_w"]),
                                       _lib.ptr(x), _lib.ptr(ids), _lib.ptr(tw), _lib.ptr(out),
                                       _lib.ptr(state["workspace"]), state["workspace_bytes"], T, _stream()),
                   "msk_moe_forward")
    else:
        ids = torch.empty((T, cfg.top_k), dtype=torch.int32, device=x.device)
        tw = torch.empty((T, cfg.top_k), dtype=torch.float32, device=x.device)
        _lib.check(lib.msk_moe_forward_logits(ctypes.byref(cfg), _lib.ptr(state["packed13"]), _lib.ptr(state["packed2"]),
                                              _lib.ptr(state["gs13"]), _lib.ptr(state["gs2"]),
                                              _lib.ptr(state["post_norm_w"]), _lib.ptr(x), _lib.ptr(logits),
                                              _lib.ptr(state["route_bias"]), _lib.ptr(ids), _lib.ptr(tw), _lib.ptr(out),
                                              _lib.ptr(state["workspace"]), state["workspace_bytes"], T, _stream()),
                   "msk_moe_forward_logits")
    if return_routing:
        return out, ids, tw
    return out


class GraphedStep:
    """kernel_fn for a fixed token count, captured once into a CUDA graph over static device buffers
    (how the decode layer consumes the module: its steps are graph replays). Calling it copies the
    inputs into the static buffers, replays the graph on the current stream and returns the static
    output tensor, which the next call overwrites. Device inputs are copied tensor by tensor; host
    inputs are first packed into one pinned staging block (a ring of them, each guarded by an
    event) so that they reach the device in a single asynchronous copy. Inputs: hidden_states and
    either router_logits or topk_ids + topk_weights, whichever `like` holds."""

    STAGES = 4

    def __init__(self, state, like):
        self.state = state
        dev = state["packed13"].device
        self.keys = [k for k in ("hidden_states", "router_logits", "topk_ids", "topk_weights") if like.get(k) is not None]
        spans, total = {}, 0
        for k in self.keys:
            nbytes = like[k].numel() * like[k].element_size()
            spans[k] = (total, nbytes)
            total += (nbytes + 255) // 256 * 256
        self.block = torch.empty(total, dtype=torch.uint8, device=dev)
        self.static = {k: self.block[o:o + n].view(like[k].dtype).view(tuple(like[k].shape)) for k, (o, n) in spans.items()}
        self.staging = [torch.empty(total, dtype=torch.uint8).pin_memory() for _ in range(self.STAGES)]
        self.staged = [{k: b[o:o + n].view(like[k].dtype).view(tuple(like[k].shape)) for k, (o, n) in spans.items()}
                       for b in self.staging]
        self.copied = [None] * self.STAGES
        self.turn = 0
        for k in self.keys:
            self.static[k].copy_(like[k])
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):                      # warm-up outside the capture
            kernel_fn(self.static, state)
        torch.cuda.current_stream(dev).wait_stream(side)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.out = kernel_fn(self.static, state)

    def __call__(self, data):
        if all(not data[k].is_cuda for k in self.keys):
            i = self.turn
            self.turn = (i + 1) % self.STAGES
            if self.copied[i] is not None:
                self.copied[i].synchronize()               # the copy that last used this block has finished
            for k in self.keys:
                self.staged[i][k].copy_(data[k])
            self.block.copy_(self.staging[i], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
            self.copied[i] = ev
        else:
            for k in self.keys:
                self.static[k].copy_(data[k], non_blocking=True)
        self.graph.replay()
        return self.out


class HostMappedStep:
    """kernel_fn for a fixed, small token count whose inputs and output stay in pinned host memory:
    the captured kernels read hidden_states and router_logits straight from a pinned block over PCIe
    (pinned memory is device-addressable under unified addressing) and write the BF16 output rows
    straight into a pinned host tensor, so a step that starts and ends on the host has no copy
    launches around the kernel at all. At a few tokens the copies are a quarter of the step (launches
    of several microseconds each around a 45 us kernel); the reads they replace are 8 KB per token
    once, plus the logits row every CTA needs, and cost one PCIe round trip.

    step(data) copies data's host tensors into a pinned block, replays the graph captured over that
    block on the current stream and returns the pinned output tensor of that block; it holds this
    step's rows once the stream (or step.done) has been synchronised. STAGES blocks (each with its own
    graph and output) are used in turn, so the host may run ahead of the device by that many steps; a
    block is reused only after the replay that read it has finished. Needs hidden_states and
    router_logits (or topk_ids + topk_weights) in `like`."""

    STAGES = 4
    _DTYPES = {"hidden_states": torch.bfloat16, "router_logits": torch.float32, "topk_ids": torch.int32,
               "topk_weights": torch.float32}

    def __init__(self, state, like):
        self.state = state
        cfg = state["cfg"]
        dev = state["packed13"].device
        if state.get("pre_norm_w") is not None:
            raise RuntimeError("HostMappedStep: states with a pre-expert norm are not supported")
        self.routed = like.get("topk_ids") is not None
        self.keys = ["hidden_states"] + (["topk_ids", "topk_weights"] if self.routed else ["router_logits"])
        if any(like.get(k) is None for k in self.keys):
            raise RuntimeError("HostMappedStep: need hidden_states and router_logits (or topk_ids + topk_weights)")
        self.T = T = like["hidden_states"].shape[0]
        spans, total = {}, 0
        for k in self.keys:
            nbytes = like[k].numel() * torch.empty((), dtype=self._DTYPES[k]).element_size()
            spans[k] = (total, nbytes)
            total += (nbytes + 255) // 256 * 256
        self.blocks = [torch.empty(total, dtype=torch.uint8).pin_memory() for _ in range(self.STAGES)]
        self.inputs = [{k: b[o:o + n].view(self._DTYPES[k]).view(tuple(like[k].shape)) for k, (o, n) in spans.items()}
                       for b in self.blocks]
        self.outs = [torch.empty((T, cfg.hidden), dtype=torch.bfloat16).pin_memory() for _ in range(self.STAGES)]
        self.ids = torch.empty((T, cfg.top_k), dtype=torch.int32, device=dev)
        self.tw = torch.empty((T, cfg.top_k), dtype=torch.float32, device=dev)
        self.events = [None] * self.STAGES
        self.done = None
        self.turn = 0
        for inp in self.inputs:
            for k in self.keys:
                inp[k].copy_(like[k])
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):                      # warm-up outside the capture
            self._launch(0)
        torch.cuda.current_stream(dev).wait_stream(side)
        self.graphs = []
        for i in range(self.STAGES):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._launch(i)
            self.graphs.append(g)

    def _launch(self, i):
        state, inp = self.state, self.inputs[i]
        cfg, lib = state["cfg"], state["lib"].lib
        args = (ctypes.byref(cfg), _lib.ptr(state["packed13"]), _lib.ptr(state["packed2"]), _lib.ptr(state["gs13"]),
                _lib.ptr(state["gs2"]), _lib.ptr(state["post_norm_w"]), _lib.ptr(inp["hidden_states"]))
        tail = (_lib.ptr(self.outs[i]), _lib.ptr(state["workspace"]), state["workspace_bytes"], self.T, _stream())
        if self.routed:
            _lib.check(lib.msk_moe_forward(*args, _lib.ptr(inp["topk_ids"]), _lib.ptr(inp["topk_weights"]), *tail),
                       "msk_moe_forward")
        else:
            _lib.check(lib.msk_moe_forward_logits(*args, _lib.ptr(inp["router_logits"]), _lib.ptr(state["route_bias"]),
                                                  _lib.ptr(self.ids), _lib.ptr(self.tw), *tail), "msk_moe_forward_logits")

    def __call__(self, data):
        i = self.turn
        self.turn = (i + 1) % self.STAGES
        if self.events[i] is not None:
            self.events[i].synchronize()   # the replay that last used this block has finished
        for k in self.keys:
            self.inputs[i][k].copy_(data[k])
        self.graphs[i].replay()
        self.done = self.events[i] = torch.cuda.Event()
        self.done.record()
        return self.outs[i]


def kernel_fn_timed(data, state):
    """kernel_fn with CUDA events around each launch of the expert step; synchronises.
    Returns (out, [ms routing + sort, ms row copy, ms gate/up GEMM, ms down GEMM, ms combine]); the
    one-launch path for a few tokens reports the whole step under gate/up. Measuring only."""
    cfg, lib = state["cfg"], state["lib"].lib
    x = data["hidden_states"].contiguous()
    T = x.shape[0]
    ids, tw = _route(data, state, x, T)
    out = torch.empty((T, cfg.hidden), dtype=torch.bfloat16, device=x.device)
    ms = (ctypes.c_float * 5)()
    _lib.check(lib.msk_moe_forward_timed(ctypes.byref(cfg), _lib.ptr(state["packed13"]), _lib.ptr(state["packed2"]),
                                         _lib.ptr(state["gs13"]), _lib.ptr(state["gs2"]),
                                         _lib.ptr(state["post_norm_w"]), _lib.ptr(x), _lib.ptr(ids), _lib.ptr(tw),
                                         _lib.ptr(out), _lib.ptr(state["workspace"]), state["workspace_bytes"], T,
                                         _stream(), ms), "msk_moe_forward_timed")
    return out, list(ms)


def plan(state, T):
    """(token tile N, path, flat shares, grid) that kernel_fn uses for T tokens (see msk_moe_plan)."""
    out = (ctypes.c_int * 4)()
    _lib.check(state["lib"].lib.msk_moe_plan(ctypes.byref(state["cfg"]), T, out), "msk_moe_plan")
    return tuple(out)


def export_weights(state):
    """Inverse of the prepare-time repack: the original codes and scale bytes, bit for bit."""
    cfg, lib = state["cfg"], state["lib"].lib
    dev = state["packed13"].device
    E, H, I = cfg.local_count, cfg.hidden, cfg.inter
    w13 = torch.empty((E, 2 * I, H // 2), dtype=torch.uint8, device=dev)
    w13_sf = torch.empty((E, 2 * I, H // 16), dtype=torch.uint8, device=dev)
    w2 = torch.empty((E, H, I // 2), dtype=torch.uint8, device=dev)
    w2_sf = torch.empty((E, H, I // 16), dtype=torch.uint8, device=dev)
    _lib.check(lib.msk_moe_unpack(ctypes.byref(cfg), _lib.ptr(state["packed13"]), _lib.ptr(state["packed2"]),
                                  _lib.ptr(w13), _lib.ptr(w13_sf), _lib.ptr(w2), _lib.ptr(w2_sf), _stream()),
               "msk_moe_unpack")
    return {"w13": w13, "w13_sf": w13_sf, "w2": w2, "w2_sf": w2_sf}


def dequant_packed(state):
    """BF16 e2m1*e4m3 matrices decoded on the device from the packed tiles (test hook)."""
    cfg, lib = state["cfg"], state["lib"].lib
    dev = state["packed13"].device
    E, H, I = cfg.local_count, cfg.hidden, cfg.inter
    dq13 = torch.empty((E, 2 * I, H), dtype=torch.bfloat16, device=dev)
    dq2 = torch.empty((E, H, I), dtype=torch.bfloat16, device=dev)
    _lib.check(lib.msk_moe_dequant_packed(ctypes.byref(cfg), _lib.ptr(state["packed13"]), _lib.ptr(state["packed2"]),
                                          _lib.ptr(dq13), _lib.ptr(dq2), _stream()), "msk_moe_dequant_packed")
    return dq13, dq2


def read_status(state):
    """Device status word (0 = every bounded wait completed). Synchronises; not for the timed path."""
    out = ctypes.c_int(-1)
    _lib.check(state["lib"].lib.msk_moe_read_status(_lib.ptr(state["workspace"]), ctypes.byref(out), _stream()),
               "msk_moe_read_status")
    return out.value


def workspace_views(state, T):
    """cnt, off, perm, inv, inter, y of the last kernel_fn call with T tokens (copies)."""
    cfg, lib = state["cfg"], state["lib"].lib
    ws = state["workspace"]
    base = ws.data_ptr()

    def view(which, nbytes, dtype):
        p = ctypes.c_void_p()
        _lib.check(lib.msk_moe_workspace_view(ctypes.byref(cfg), _lib.ptr(ws), which, ctypes.byref(p)), "workspace_view")
        o = p.value - base
        return ws[o:o + nbytes].view(dtype).clone()

    E, k = cfg.local_count, cfg.top_k
    cnt = view(0, E * 4, torch.int32)
    off = view(1, (E + 1) * 4, torch.int32)
    R = int(off[-1].item())
    perm = view(2, T * k * 4, torch.int32)
    inv = view(3, T * k * 4, torch.int32)
    inter = view(4, R * cfg.inter * 2, torch.float16).view(R, cfg.inter)
    n_tile = plan(state, T)[0]
    if n_tile == 128:      # the wide token tile keeps y in BF16
        y = view(5, R * cfg.hidden * 2, torch.bfloat16).view(R, cfg.hidden)
    else:
        y = view(5, R * cfg.hidden * 4, torch.float32).view(R, cfg.hidden)
    return {"cnt": cnt, "off": off, "perm": perm, "inv": inv, "inter": inter, "y": y}


def trace_stamps(state):
    """(stamps int64 [2, 256, 16], events int64 [2, 6, 128]) of the last step's GEMM launches
    (prepare(trace=1)): per-CTA %globaltimer stamps, and one CTA's event list per role (dequant
    thread, MMA issuer, weight producer, epilogue thread, gather warp; only in a library built with
    MSK_TRACE_DETAIL), each event = ns << 8 | code."""
    cfg, lib = state["cfg"], state["lib"].lib
    ws = state["workspace"]
    p = ctypes.c_void_p()
    _lib.check(lib.msk_moe_workspace_view(ctypes.byref(cfg), _lib.ptr(ws), 6, ctypes.byref(p)), "workspace_view")
    o = p.value - ws.data_ptr()
    words = 256 * 16 + 3 * 256
    t = ws[o:o + 2 * words * 8].view(torch.int64).view(2, words).clone()
    return t[:, :256 * 16].reshape(2, 256, 16), t[:, 256 * 16:].reshape(2, 6, 128)


class L2Sweep:
    """Cold-cache timing aid: sweep() reads a buffer larger than L2 (256 MiB) on the current stream."""

    def __init__(self, device, nbytes=256 << 20):
        self.buf = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        self.sink = torch.zeros(4, dtype=torch.int32, device=device)
        self.lib = _lib.load()

    def sweep(self):
        _lib.check(self.lib.msk_l2_sweep(_lib.ptr(self.buf), self.buf.numel(), _lib.ptr(self.sink), _stream()), "msk_l2_sweep")


def bw_probe(nbytes=1 << 30, stages=5, stage_bytes=36864, num_ctas=0, skip_release=0, device=None):
    """HBM streaming probe (msk_bw_probe). Returns (GB/s, device status): status 1 means a bounded
    wait inside the kernel gave up (what skip_release > 0 provokes on purpose)."""
    lib = _lib.load()
    dev = device or torch.device("cuda", torch.cuda.current_device())
    src = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    sink = torch.zeros(2, dtype=torch.int32, device=dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    _lib.check(lib.msk_bw_probe(_lib.ptr(src), nbytes, stages, stage_bytes, num_ctas, _lib.ptr(sink), skip_release,
                                _stream()), "msk_bw_probe")
    e1.record()
    torch.cuda.synchronize(dev)
    return nbytes / (e0.elapsed_time(e1) * 1e-3) / 1e9, int(sink[1].item())


def attrs(which, token_tile=16):
    """(registers, static smem, max dynamic smem, local bytes) of a kernel; see msk_moe_attrs."""
    out = (ctypes.c_int * 4)()
    _lib.check(_lib.load().msk_moe_attrs(which, token_tile, out), "msk_moe_attrs")
    return tuple(out)
