"""GPU parity tests: the CUDA path (through the C ABI) against the CPU oracle.

Bars: bit-exact for codes, scale bytes, ids, counts, offsets, permutation; expert outputs
within max-abs error / max-abs reference <= 1e-2 of the FP32 oracle.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = 1e-2  # max|out - ref| / max|ref|, the tolerance the north star states


def _rel(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


def _mods():
    import muse_moe_w4a16 as m
    from muse_moe_w4a16 import inputs, _lib
    from oracle import moe_oracle as orc
    return m, inputs, _lib, orc


def _adversarial_weights(H, I, E, dev, seed=3):
    """Random codes (all 16, sign bits included) and scale bytes covering zero, subnormal,
    normal and the largest finite E4M3 values."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    special = torch.tensor([0x00, 0x01, 0x07, 0x08, 0x38, 0x40, 0x7E, 0x30, 0x3F, 0x20], dtype=torch.uint8)

    def mk(rows, K):
        codes = torch.randint(0, 256, (E, rows, K // 2), generator=g, dtype=torch.uint8)
        sf = special[torch.randint(0, len(special), (E, rows, K // 16), generator=g)]
        return codes.to(dev), sf.to(dev)

    w13, w13_sf = mk(2 * I, H)
    w2, w2_sf = mk(H, I)
    return {"w13": w13, "w13_sf": w13_sf.view(torch.float8_e4m3fn), "w13_gs": torch.full((E,), 1e-3, device=dev),
            "w2": w2, "w2_sf": w2_sf.view(torch.float8_e4m3fn), "w2_gs": torch.full((E,), 1e-3, device=dev)}


def test_repack_is_lossless_and_decode_matches_oracle(cuda_dev):
    m, inputs, _lib, orc = _mods()
    H, I, E = 512, 256, 3
    w = _adversarial_weights(H, I, E, cuda_dev)
    st = m.prepare(w, max_tokens=8)
    back = m.export_weights(st)
    for k in ("w13", "w2"):
        assert torch.equal(back[k], w[k])
    for k in ("w13_sf", "w2_sf"):
        assert torch.equal(back[k], w[k].view(torch.uint8))
    dq13, dq2 = m.dequant_packed(st)
    torch.cuda.synchronize()
    for dq, c, s in ((dq13, w["w13"], w["w13_sf"]), (dq2, w["w2"], w["w2_sf"])):
        ref = orc.dequant(c.cpu().numpy(), s.view(torch.uint8).cpu().numpy())
        got = dq.float().cpu().numpy()
        assert np.array_equal(got, ref)  # e2m1 * e4m3 is exact in BF16


def test_decode_all_codes_times_all_scale_bytes(cuda_dev):
    """Known-answer sweep: 16 codes x 256 scale bytes (NaN bytes included)."""
    m, inputs, _lib, orc = _mods()
    H, I, E = 512, 256, 1
    # w13 rows: row r uses scale byte r % 256 everywhere; codes cycle through all 16
    codes = (torch.arange(H // 2) % 8).to(torch.uint8)
    codes = (2 * codes) | ((2 * codes + 1) << 4)          # nibble pairs (0,1),(2,3)...(14,15)
    w13 = codes.repeat(2 * I, 1).unsqueeze(0).contiguous()
    sf13 = (torch.arange(2 * I) % 256).to(torch.uint8).unsqueeze(1).repeat(1, H // 16).unsqueeze(0).contiguous()
    w2 = torch.zeros((1, H, I // 2), dtype=torch.uint8)
    sf2 = torch.zeros((1, H, I // 16), dtype=torch.uint8)
    w = {"w13": w13.to(cuda_dev), "w13_sf": sf13.to(cuda_dev), "w13_gs": torch.ones(1, device=cuda_dev),
         "w2": w2.to(cuda_dev), "w2_sf": sf2.to(cuda_dev), "w2_gs": torch.ones(1, device=cuda_dev)}
    st = m.prepare(w, max_tokens=8)
    dq13, _ = m.dequant_packed(st)
    got = dq13[0].float().cpu().numpy()
    ref = orc.dequant(w13[0].numpy(), sf13[0].numpy())
    assert np.array_equal(np.isnan(got), np.isnan(ref))
    ok = ~np.isnan(ref)
    assert np.array_equal(got[ok], ref[ok])


@pytest.mark.parametrize("T,E,k,mode", [(1, 128, 8, "softmax_topk"), (37, 128, 8, "softmax_topk"),
                                        (64, 256, 8, "sigmoid_bias"), (5, 8, 2, "softmax_topk"),
                                        (300, 512, 16, "sigmoid_bias")])
def test_route_topk_bit_exact_ids(cuda_dev, T, E, k, mode):
    m, inputs, _lib, orc = _mods()
    lib = _lib.load()
    g = torch.Generator(device="cpu").manual_seed(T * 131 + E)
    logits = torch.randn((T, E), generator=g)
    logits[:, : E // 4] = logits[:, E // 4: E // 2][:, : E // 4]  # exact ties between experts
    bias = torch.randn((E,), generator=g) * 0.1 if mode == "sigmoid_bias" else None
    cfg = _lib.MskMoeCfg(hidden=512, inter=256, n_experts=E, local_start=0, local_count=min(E, 256), top_k=k,
                         routing_mode=m._MODES[mode], route_scale=0.1767766952966369, post_norm_eps=1e-8,
                         max_tokens=T)
    ld = logits.to(cuda_dev)
    bd = None if bias is None else bias.to(cuda_dev)
    ids = torch.empty((T, k), dtype=torch.int32, device=cuda_dev)
    tw = torch.empty((T, k), dtype=torch.float32, device=cuda_dev)
    _lib.check(lib.msk_moe_route(ctypes.byref(cfg), _lib.ptr(ld), _lib.ptr(bd), _lib.ptr(ids), _lib.ptr(tw), T,
                                 ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)), "route")
    torch.cuda.synchronize()
    rid, rw = orc.route_topk(logits, k, mode, bias)
    got = ids.cpu()
    if mode == "sigmoid_bias":
        # The score sigmoid(l * scale) + bias is evaluated by two exp implementations (device, host)
        # that may differ in the last bits. An id may therefore differ from the oracle's only where the
        # two candidates' scores are within 4 ulp of each other ("tie-risk"); anything else fails.
        sel = (torch.sigmoid(logits * 0.1767766952966369) + bias).numpy()
        a, b = got.numpy(), rid.numpy()
        rows, slots = np.nonzero(a != b)
        for r, c in zip(rows, slots):
            sa, sb = sel[r, a[r, c]], sel[r, b[r, c]]
            assert abs(float(sa) - float(sb)) <= 4 * float(np.spacing(np.float32(max(abs(sa), abs(sb))))), (r, c, sa, sb)
        assert len(set(rows.tolist())) <= max(1, T // 20)   # near-ties are rare on random logits
        same = torch.from_numpy(~np.isin(np.arange(T), rows))
        assert torch.allclose(tw.cpu()[same], rw[same], rtol=1e-5, atol=1e-7)
    else:
        assert torch.equal(got, rid)
        assert torch.allclose(tw.cpu(), rw, rtol=1e-5, atol=1e-7)


@pytest.mark.parametrize("T,E,k,lo,nloc", [(1, 128, 8, 0, 128), (7, 128, 8, 0, 128), (256, 128, 8, 0, 128),
                                           (100, 256, 8, 64, 32), (8192, 128, 8, 0, 128), (33, 8, 2, 0, 8),
                                           (4097, 256, 8, 32, 32)])
def test_sort_bit_exact(cuda_dev, T, E, k, lo, nloc):
    m, inputs, _lib, orc = _mods()
    lib = _lib.load()
    g = torch.Generator(device="cpu").manual_seed(T + 7 * E)
    ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(min(T, 512))]).to(torch.int32)
    if T > 512:
        ids = ids.repeat((T + 511) // 512, 1)[:T].contiguous()
        ids = (ids + torch.arange(T, dtype=torch.int32).unsqueeze(1) * 5) % E
    ids[0, 0] = -1  # a dropped entry, as the decode layer's local-id convention produces
    cfg = _lib.MskMoeCfg(hidden=512, inter=256, n_experts=E, local_start=lo, local_count=nloc, top_k=k, max_tokens=T)
    d = ids.to(cuda_dev)
    cnt = torch.zeros(nloc, dtype=torch.int32, device=cuda_dev)
    off = torch.zeros(nloc + 1, dtype=torch.int32, device=cuda_dev)
    perm = torch.full((T * k,), -7, dtype=torch.int32, device=cuda_dev)
    inv = torch.full((T * k,), -7, dtype=torch.int32, device=cuda_dev)
    _lib.check(lib.msk_moe_sort(ctypes.byref(cfg), _lib.ptr(d), T, _lib.ptr(cnt), _lib.ptr(off), _lib.ptr(perm),
                                _lib.ptr(inv), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)), "sort")
    torch.cuda.synchronize()
    rc, ro, rp, ri = orc.sort_routes(ids.numpy(), lo, nloc)
    R = int(ro[-1])
    assert np.array_equal(cnt.cpu().numpy(), rc)
    assert np.array_equal(off.cpu().numpy(), ro)
    assert np.array_equal(perm.cpu().numpy()[:R], rp)
    assert np.array_equal(inv.cpu().numpy(), ri)


def _run_forward(m, inputs, orc, dev, H, I, E, k, T, seed, post_norm=False, logits_kind="normal", lo=0, nloc=None,
                 **prep):
    nloc = E if nloc is None else nloc
    w = inputs.make_weights(H, I, nloc, seed, dev, post_norm=post_norm)
    st = m.prepare(w, local_start=lo, n_experts=E, top_k=k, max_tokens=max(T, 1), **prep)
    g = torch.Generator(device=dev).manual_seed(seed + 99)
    x = torch.randn((T, H), generator=g, device=dev).to(torch.bfloat16)
    logits = inputs.make_logits(T, E, logits_kind, seed, dev)
    out, ids, tw = m.kernel_fn({"hidden_states": x, "router_logits": logits}, st, return_routing=True)
    torch.cuda.synchronize()
    assert m.read_status(st) == 0
    ref, parts = orc.moe_forward(x, ids, tw, w, local_start=lo, return_parts=True)
    views = m.workspace_views(st, T)
    return out, ref, parts, views, st, (x, ids, tw, w)


def _check_forward(out, ref, parts, views):
    assert np.array_equal(views["cnt"].cpu().numpy(), parts["cnt"])
    assert np.array_equal(views["off"].cpu().numpy(), parts["off"])
    R = int(parts["off"][-1])
    assert np.array_equal(views["perm"].cpu().numpy()[:R], parts["perm"])
    assert np.array_equal(views["inv"].cpu().numpy(), parts["inv"])
    assert _rel(views["inter"], parts["inter"]) <= TOL
    assert _rel(views["y"], parts["y"]) <= TOL
    assert _rel(out, parts["out_fp32"]) <= TOL


def test_forward_tiny_config0(cuda_dev):
    """Config 0: H=512, I=256, E=8, top-2, T=4, router weight in the module."""
    m, inputs, _lib, orc = _mods()
    H, I, E, k, T = 512, 256, 8, 2, 4
    w = inputs.make_weights(H, I, E, 0, cuda_dev)
    g = torch.Generator(device=cuda_dev).manual_seed(0)
    x = torch.randn((T, H), generator=g, device=cuda_dev).to(torch.bfloat16)
    w["router"] = torch.randn((E, H), generator=g, device=cuda_dev) * 0.02
    st = m.prepare(w, n_experts=E, top_k=k, max_tokens=T)
    out, ids, tw = m.kernel_fn({"hidden_states": x}, st, return_routing=True)
    torch.cuda.synchronize()
    assert m.read_status(st) == 0
    logits = orc.router_logits(x.cpu(), w["router"].cpu())
    rid, rw = orc.route_topk(logits, k)
    assert torch.equal(ids.cpu(), rid)
    assert torch.allclose(tw.cpu(), rw, rtol=1e-4, atol=1e-6)
    ref, parts = orc.moe_forward(x, ids, tw, w, return_parts=True)
    _check_forward(out, ref, parts, m.workspace_views(st, T))


@pytest.mark.parametrize("T,tile,path,post", [(1, 0, 0, False), (5, 16, 0, True), (5, 16, 1, False), (5, 16, 2, True),
                                              (40, 32, 1, False), (70, 64, 1, True), (300, 128, 1, False),
                                              (9, 16, 0, True), (9, 16, 1, True), (600, 0, 1, True), (300, 128, 1, True),
                                              (32, 16, 0, False), (32, 32, 2, True), (17, 32, 0, True), (32, 16, 1, True)])
def test_forward_small_shapes(cuda_dev, T, tile, path, post):
    """Every token tile and, for a few tokens, every path (0 one launch, 1 chain of launches, 2 row
    copy + routing gate/up kernel + combining down kernel)."""
    m, inputs, _lib, orc = _mods()
    out, ref, parts, views, st, _ = _run_forward(m, inputs, orc, cuda_dev, 512, 256, 8, 2, T, seed=T, post_norm=post,
                                                 token_tile=tile, decode_path=path or 3, flat_shares=1)
    if T <= 32:
        assert m.plan(st, T)[1] == path
    _check_forward(out, ref, parts, views)


@pytest.mark.parametrize("T,path,ctas,post", [(1, 0, 0, False), (1, 0, 37, True), (1, 2, 0, True), (1, 1, 0, False),
                                              (3, 0, 5, True), (3, 2, 148, False), (8, 0, 0, True), (8, 2, 37, False),
                                              (8, 1, 100, True), (32, 0, 0, True), (32, 0, 111, False), (32, 2, 0, True),
                                              (20, 0, 1, False), (2, 0, 148, True)])
def test_forward_few_token_paths_and_grids(cuda_dev, T, path, ctas, post):
    """Few tokens: the weight stream is cut into equal shares per CTA, so units are summed from pieces
    whose cut points move with the grid size; the kernels route, sort and combine themselves (paths 0
    and 2). Every combination must match the oracle, give the same bits with the routing passed in
    instead of the logits, and stay within rounding of the chain of launches."""
    m, inputs, _lib, orc = _mods()
    H, I, E, k = 1024, 512, 16, 4
    out, ref, parts, views, st, (x, ids, tw, w) = _run_forward(m, inputs, orc, cuda_dev, H, I, E, k, T, seed=60 + T,
                                                               post_norm=post, decode_path=path or 3, num_ctas=ctas,
                                                               flat_shares=1)
    plan = m.plan(st, T)
    assert plan[1] == path and plan[2] == (0 if path == 0 else 1) and plan[3] == (ctas or 148)
    _check_forward(out, ref, parts, views)
    again = m.kernel_fn({"hidden_states": x, "topk_ids": ids, "topk_weights": tw}, st)
    assert torch.equal(again, out)
    chain = m.prepare(w, n_experts=E, top_k=k, max_tokens=T, decode_path=1, token_tile=16, num_ctas=3, flat_shares=1)
    other = m.kernel_fn({"hidden_states": x, "topk_ids": ids, "topk_weights": tw}, chain)
    assert _rel(out, other) <= 8e-3   # same products, other cut points: a bf16 ulp or two of the output
    torch.cuda.synchronize()
    assert m.read_status(st) == 0 and m.read_status(chain) == 0


def test_forward_decode_shape_T1_and_T8(cuda_dev):
    """Config 1/2 shape with fewer experts resident (E=16 of the 4096 x 1536 experts)."""
    m, inputs, _lib, orc = _mods()
    for T, path in ((1, 0), (8, 0), (1, 2), (8, 2), (8, 1)):
        out, ref, parts, views, st, _ = _run_forward(m, inputs, orc, cuda_dev, 4096, 1536, 16, 8, T, seed=10 + T,
                                                     decode_path=path or 3, flat_shares=1)
        assert m.plan(st, T)[:3] == (16, path, 0 if path == 0 else 1)
        _check_forward(out, ref, parts, views)


def test_ep_combine_kernel_matches_rank_order_sum(cuda_dev):
    """msk_ep_combine against the same rank-order FP32 sum in torch (bit-exact: same order, same
    arithmetic); rows of ranks a token does not route to are never read."""
    from muse_moe_w4a16 import ep

    n, T, H, k, per = 4, 300, 512, 3, 8
    g = torch.Generator(device=cuda_dev).manual_seed(9)
    back = torch.randn((n, T, H), generator=g, device=cuda_dev).to(torch.bfloat16)
    ids = torch.stack([torch.randperm(n * per, generator=g, device=cuda_dev)[:k] for _ in range(T)]).to(torch.int32)
    ids[0] = -1  # a token with no route anywhere sums to zero
    mask = ep.route_mask(ids, n, per)
    poisoned = back.clone()
    poisoned[~mask] = float("nan")
    got = ep.combine_partials(poisoned, ids, per)
    want = ep.combine_partials(back.cpu(), ids.cpu(), per)
    assert torch.equal(got.cpu(), want)
    assert float(got[0].float().abs().max()) == 0.0
    own = ep.combine_partials(poisoned, ids, per, self_rank=1, self_rows=back[1].contiguous())
    assert torch.equal(own, got)


@pytest.mark.parametrize("tile,path", [(16, 0), (16, 1), (16, 2), (32, 0)])
def test_forward_local_range_negative_ids_and_empty_tokens(cuda_dev, tile, path):
    """Experts [4, 12) of 16 resident: routes outside the range and negative ids are dropped (the
    reference's filter, muse_moe_w4a16/cuda/moe.cu:347-350); a token left without any route is zero."""
    m, inputs, _lib, orc = _mods()
    H, I, E, k, T, lo, nloc = 512, 256, 16, 4, 6, 4, 8
    w = inputs.make_weights(H, I, nloc, 31, cuda_dev, post_norm=True)
    st = m.prepare(w, local_start=lo, n_experts=E, top_k=k, max_tokens=T, token_tile=tile, decode_path=path or 3,
                   flat_shares=1)
    g = torch.Generator(device=cuda_dev).manual_seed(5)
    x = torch.randn((T, H), generator=g, device=cuda_dev).to(torch.bfloat16)
    ids = torch.stack([torch.randperm(E, generator=g, device=cuda_dev)[:k] for _ in range(T)]).to(torch.int32)
    ids[1] = torch.tensor([0, 1, 14, 15], dtype=torch.int32)      # nothing local
    ids[2, 0] = -1
    ids[3] = -1                                                   # no route at all
    tw = torch.rand((T, k), generator=g, device=cuda_dev)
    out = m.kernel_fn({"hidden_states": x, "topk_ids": ids, "topk_weights": tw}, st)
    torch.cuda.synchronize()
    assert m.read_status(st) == 0
    ref, parts = orc.moe_forward(x, ids, tw, w, local_start=lo, return_parts=True)
    _check_forward(out, ref, parts, m.workspace_views(st, T))
    assert float(out[1].float().abs().max()) == 0.0 and float(out[3].float().abs().max()) == 0.0


@pytest.mark.parametrize("T", [1, 8, 40])
def test_forward_is_deterministic_and_graph_capturable(cuda_dev, T):
    """Same inputs, same bits: across calls, and between an eager call and a CUDA-graph replay."""
    m, inputs, _lib, orc = _mods()
    H, I, E, k = 1024, 512, 16, 4
    w = inputs.make_weights(H, I, E, 41, cuda_dev, post_norm=True)
    st = m.prepare(w, n_experts=E, top_k=k, max_tokens=T)
    g = torch.Generator(device=cuda_dev).manual_seed(6)
    data = {"hidden_states": torch.randn((T, H), generator=g, device=cuda_dev).to(torch.bfloat16),
            "router_logits": torch.randn((T, E), generator=g, device=cuda_dev)}
    first = m.kernel_fn(data, st).clone()
    for _ in range(3):
        assert torch.equal(m.kernel_fn(data, st), first)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        m.kernel_fn(data, st)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        captured = m.kernel_fn(data, st)
    for _ in range(2):
        captured.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(captured, first)
    assert m.read_status(st) == 0


def test_forward_zero_tokens_and_state_deepcopy(cuda_dev):
    import copy

    m, inputs, _lib, orc = _mods()
    H, I, E, k = 512, 256, 8, 2
    w = inputs.make_weights(H, I, E, 43, cuda_dev)
    st = m.prepare(w, n_experts=E, top_k=k, max_tokens=4)
    empty = m.kernel_fn({"hidden_states": torch.empty((0, H), dtype=torch.bfloat16, device=cuda_dev),
                         "topk_ids": torch.empty((0, k), dtype=torch.int32, device=cuda_dev),
                         "topk_weights": torch.empty((0, k), device=cuda_dev)}, st)
    assert tuple(empty.shape) == (0, H)
    st2 = copy.deepcopy(st)
    g = torch.Generator(device=cuda_dev).manual_seed(8)
    data = {"hidden_states": torch.randn((3, H), generator=g, device=cuda_dev).to(torch.bfloat16),
            "router_logits": torch.randn((3, E), generator=g, device=cuda_dev)}
    assert torch.equal(m.kernel_fn(data, st), m.kernel_fn(data, st2))


@pytest.mark.parametrize("T,E,k,lo,nloc", [(8192, 8, 2, 0, 8), (4096, 16, 4, 4, 8)])
def test_forward_many_entries_sorted_on_several_ctas(cuda_dev, T, E, k, lo, nloc):
    """From 16384 routed entries on, the stable sort runs on several CTAs (count, scan, scatter); the
    tables must still equal the oracle's stable sort bit for bit, with and without a local range."""
    m, inputs, _lib, orc = _mods()
    out, ref, parts, views, st, _ = _run_forward(m, inputs, orc, cuda_dev, 512, 256, E, k, T, seed=77, post_norm=True,
                                                 lo=lo, nloc=nloc, logits_kind="zipf")
    assert T * k >= 16384
    _check_forward(out, ref, parts, views)


def test_graphed_step_with_pinned_host_inputs(cuda_dev):
    """GraphedStep (static buffers + CUDA graph) returns what kernel_fn returns, bit for bit, for
    device inputs and for pinned host inputs, call after call."""
    m, inputs, _lib, orc = _mods()
    H, I, E, k, T = 1024, 512, 16, 4, 5
    w = inputs.make_weights(H, I, E, 51, cuda_dev, post_norm=True)
    st = m.prepare(w, n_experts=E, top_k=k, max_tokens=T)
    g = torch.Generator(device=cuda_dev).manual_seed(9)
    datas = [{"hidden_states": torch.randn((T, H), generator=g, device=cuda_dev).to(torch.bfloat16),
              "router_logits": torch.randn((T, E), generator=g, device=cuda_dev)} for _ in range(3)]
    step = m.GraphedStep(st, datas[0])
    for d in datas + datas[:1]:
        want = m.kernel_fn(d, st)
        host = {key: v.cpu().pin_memory() for key, v in d.items()}
        got_dev = step(d).clone()
        got_host = step(host).clone()
        torch.cuda.synchronize()
        assert torch.equal(got_dev, want) and torch.equal(got_host, want)
    assert m.read_status(st) == 0


@pytest.mark.parametrize("T,routed", [(1, False), (5, False), (8, True), (40, False)])
def test_host_mapped_step_reads_and_writes_pinned_host_memory(cuda_dev, T, routed):
    """HostMappedStep (kernels read the inputs from, and write the output to, pinned host memory; no copy
    launches) returns what kernel_fn returns on device tensors, bit for bit, call after call and across
    its ring of blocks: one-launch path (1, 5, 8 tokens), chain (40 tokens), given ids and logits."""
    m, inputs, _lib, orc = _mods()
    H, I, E, k = 1024, 512, 16, 4
    w = inputs.make_weights(H, I, E, 52, cuda_dev, post_norm=True)
    st = m.prepare(w, n_experts=E, top_k=k, max_tokens=T)
    g = torch.Generator(device=cuda_dev).manual_seed(10 + T)
    datas = []
    for _ in range(6):
        d = {"hidden_states": torch.randn((T, H), generator=g, device=cuda_dev).to(torch.bfloat16)}
        logits = torch.randn((T, E), generator=g, device=cuda_dev)
        if routed:
            tw, ids = torch.softmax(logits, dim=-1).topk(k, dim=-1)
            d["topk_ids"], d["topk_weights"] = ids.to(torch.int32), tw.contiguous()
        else:
            d["router_logits"] = logits
        datas.append(d)
    step = m.HostMappedStep(st, {key: v.cpu() for key, v in datas[0].items()})
    for d in datas:
        want = m.kernel_fn(d, st)
        got = step({key: v.cpu() for key, v in d.items()})
        assert not got.is_cuda and got.is_pinned()
        step.done.synchronize()
        assert torch.equal(got, want.cpu())
    assert m.read_status(st) == 0


@pytest.mark.parametrize("T,tile", [(9, 0), (40, 0), (100, 16), (100, 32), (260, 32)])
def test_both_gemms_in_one_launch_behind_the_sort_gives_the_chain_bits(cuda_dev, T, tile):
    """decode_path = 4 (sort launches, then the gate/up and the down GEMM in one cooperative launch that
    hands `inter` over tile by tile, then the combine) computes every unit exactly as the chain of
    launches does: same output bits, same sort tables, status word clean, call after call."""
    m, inputs, _lib, orc = _mods()
    H, I, E, k = 1024, 512, 16, 4
    w = inputs.make_weights(H, I, E, 53, cuda_dev, post_norm=True)
    chain = m.prepare(w, n_experts=E, top_k=k, max_tokens=T, decode_path=1, token_tile=tile)
    both = m.prepare(w, n_experts=E, top_k=k, max_tokens=T, decode_path=4, token_tile=tile)
    assert m.plan(both, T)[1] == 4 and m.plan(chain, T)[1] == 1
    g = torch.Generator(device=cuda_dev).manual_seed(20 + T)
    for _ in range(3):
        d = {"hidden_states": torch.randn((T, H), generator=g, device=cuda_dev).to(torch.bfloat16),
             "router_logits": torch.randn((T, E), generator=g, device=cuda_dev)}
        want, ids_w, tw_w = m.kernel_fn(d, chain, return_routing=True)
        got, ids_g, tw_g = m.kernel_fn(d, both, return_routing=True)
        torch.cuda.synchronize()
        assert torch.equal(ids_g, ids_w) and torch.equal(tw_g, tw_w)
        assert torch.equal(got, want)
        vw, vg = m.workspace_views(chain, T), m.workspace_views(both, T)
        for key in ("cnt", "off", "perm", "inv"):
            assert torch.equal(vg[key], vw[key]), key
    assert m.read_status(both) == 0 and m.read_status(chain) == 0


def test_okc_ext_runs_the_decode_layer_call_site(cuda_dev):
    """The decode layer's call (muse_decode_layer/py/06_kernel_fn.py:140-149): local ids with -1 for
    another GPU's expert, lo = 0, an output slice filled in place, in chunks."""
    m, inputs, _lib, orc = _mods()
    from muse_moe_w4a16.compat import OkcExt

    H, I, nloc, k, T = 1024, 512, 8, 4, 11
    w = inputs.make_weights(H, I, nloc, 61, cuda_dev, post_norm=True)
    st = m.prepare(w, local_start=0, n_experts=nloc, top_k=k, max_tokens=8)
    ext = OkcExt(st)
    g = torch.Generator(device=cuda_dev).manual_seed(4)
    x = torch.randn((T, H), generator=g, device=cuda_dev).to(torch.bfloat16)
    lids = torch.randint(-1, nloc, (T, k), generator=g, device=cuda_dev, dtype=torch.int32)
    wts = torch.rand((T, k), generator=g, device=cuda_dev)
    out = torch.full((T, H), float("nan"), dtype=torch.bfloat16, device=cuda_dev)
    ext.okc_set_pdl(1)
    for m0 in range(0, T, 8):
        m1 = min(T, m0 + 8)
        ext.okc_run(None, None, x[m0:m1], lids[m0:m1], wts[m0:m1], out[m0:m1], 0, nloc, 148)
    torch.cuda.synchronize()
    ref = orc.moe_forward(x, lids, wts, w).float()
    assert _rel(out, ref) <= TOL
    assert len(ext.okc_attrs()) == 6
    with pytest.raises(RuntimeError):
        ext.okc_run(None, None, x[:1], lids[:1], wts[:1], out[:1], 1, nloc, 148)
    with pytest.raises(RuntimeError):
        ext.okc_run(None, None, x[:1], lids[:1], wts[:1], out[:1], 0, nloc, 132)   # a grid it was not prepared for
    # without programmatic dependent launch the chain of launches gives the same bits
    ext.okc_set_pdl(0)
    out2 = torch.empty_like(out)
    for m0 in range(0, T, 8):
        m1 = min(T, m0 + 8)
        ext.okc_run(None, None, x[m0:m1], lids[m0:m1], wts[m0:m1], out2[m0:m1], 0, nloc, 148)
    torch.cuda.synchronize()
    assert torch.equal(out2, out)


@pytest.mark.parametrize("T,given_ids", [(3, False), (7, True), (40, True), (300, False), (600, True)])
def test_forward_with_pre_expert_norm(cuda_dev, T, given_ids):
    """weights["pre_norm_w"]: the layer callers' pre-expert RMS norm (eps 1e-5, x (1 + g)) fused into
    the row-copy kernel, for every token-tile width; routing still sees the un-normed logits."""
    m, inputs, _lib, orc = _mods()
    H, I, E, k = 1024, 512, 8, 2
    w = inputs.make_weights(H, I, E, 71, cuda_dev, post_norm=True)
    g = torch.Generator(device=cuda_dev).manual_seed(12)
    w["pre_norm_w"] = (torch.randn((H,), generator=g, device=cuda_dev) * 0.1).to(torch.bfloat16)
    st = m.prepare(w, n_experts=E, top_k=k, max_tokens=T)
    x = (torch.randn((T, H), generator=g, device=cuda_dev) * 3.0).to(torch.bfloat16)
    logits = torch.randn((T, E), generator=g, device=cuda_dev)
    out, ids, tw = m.kernel_fn({"hidden_states": x, "router_logits": logits}, st, return_routing=True)
    if given_ids:
        out = m.kernel_fn({"hidden_states": x, "topk_ids": ids, "topk_weights": tw}, st)
    torch.cuda.synchronize()
    assert m.read_status(st) == 0
    rid, _ = orc.route_topk(logits.cpu(), k)
    assert torch.equal(ids.cpu(), rid)
    ref, parts = orc.moe_forward(x, ids, tw, w, return_parts=True)
    _check_forward(out, ref, parts, m.workspace_views(st, T))
    plain = dict(w)
    del plain["pre_norm_w"]
    assert _rel(out, orc.moe_forward(x, ids, tw, plain).float()) > 0.05   # the norm is not a no-op here


@pytest.mark.parametrize("T", [64, 8192])
def test_full_size_properties(cuda_dev, T):
    """Benchmark-size shapes (H4096 I1536 E128 top-8; T = 64 decode sweep point, T = 8192 prefill),
    where the CPU oracle would take minutes: properties that hold whatever the size.
    (1) A token's output does not depend on where the token sits: permuting the tokens permutes
    the output rows, bit for bit. (2) Halving the top-k weights halves the output exactly.
    (3) Tokens whose ids are all -1 come out zero and leave the other tokens' rows untouched."""
    m, inputs, _lib, orc = _mods()
    s = inputs.SHAPES["decode"]
    H, I, E, k = s["H"], s["I"], s["E"], s["k"]
    w = inputs.make_weights_random_bytes(H, I, E, 5, cuda_dev)
    st = m.prepare(w, n_experts=E, top_k=k, max_tokens=T)
    data, _ = inputs.make_inputs("prefill" if T > 256 else "decode", T, 3, cuda_dev)
    x, logits = data["hidden_states"], data["router_logits"]
    out, ids, tw = m.kernel_fn({"hidden_states": x, "router_logits": logits}, st, return_routing=True)
    out = out.clone()
    g = torch.Generator(device=cuda_dev).manual_seed(1)
    p = torch.randperm(T, generator=g, device=cuda_dev)
    out_p = m.kernel_fn({"hidden_states": x[p].contiguous(), "router_logits": logits[p].contiguous()}, st)
    assert torch.equal(out_p, out[p])
    half = m.kernel_fn({"hidden_states": x, "topk_ids": ids, "topk_weights": tw * 0.5}, st)
    assert torch.equal(half.float() * 2.0, out.float())
    ids2 = ids.clone()
    ids2[::7] = -1
    z = m.kernel_fn({"hidden_states": x, "topk_ids": ids2, "topk_weights": tw}, st)
    assert float(z[::7].float().abs().max()) == 0.0
    keep = torch.ones(T, dtype=torch.bool, device=cuda_dev)
    keep[::7] = False
    assert torch.equal(z[keep], out[keep])
    torch.cuda.synchronize()
    assert m.read_status(st) == 0


def _oracle_rows_of_tokens(orc, w, x, ids, tw, sel, post_norm=False):
    """Oracle evaluation of the tokens `sel` of a larger call: all of their experts (a dense local
    table over the touched ones). Returns (out bf16 [len(sel), H], parts, entry map): parts as
    orc.moe_forward returns them, and for every oracle row q' the (token index in sel, slot) it is."""
    sel_l = sel.tolist()
    sub_ids = ids[sel].cpu()
    touched = sorted(set(int(v) for v in sub_ids.flatten().tolist() if v >= 0))
    remap = {e: j for j, e in enumerate(touched)}
    lids = torch.tensor([[remap.get(int(v), -1) for v in row] for row in sub_ids.tolist()], dtype=torch.int32)

    def take(t):   # fp8 tensors are indexed through their bytes
        if t.dtype == torch.float8_e4m3fn:
            return t.view(torch.uint8)[touched].view(torch.float8_e4m3fn).cpu()
        return t[touched].cpu()

    sub = {key: take(w[key]) for key in ("w13", "w13_sf", "w13_gs", "w2", "w2_sf", "w2_gs")}
    if post_norm:
        sub["post_norm_w"] = w["post_norm_w"].cpu()
    ref, parts = orc.moe_forward(x[sel].cpu(), lids, tw[sel].cpu(), sub, return_parts=True)
    return ref, parts, sel_l


@pytest.mark.parametrize("T", [64, 8192])
def test_full_size_outputs_match_oracle_on_sampled_tokens(cuda_dev, T):
    """The benchmarked configurations themselves (H4096 I1536 E128 top-8; T = 64 with the 16-token
    tile, T = 8192 Zipf-routed with the 128-token tile and 16 K stages): eight tokens of the real
    output, and their rows of `inter` and `y` in the workspace, against the oracle evaluated on all
    of those tokens' experts."""
    m, inputs, _lib, orc = _mods()
    s = inputs.SHAPES["decode"]
    H, I, E, k = s["H"], s["I"], s["E"], s["k"]
    w = inputs.make_weights_random_bytes(H, I, E, 5, cuda_dev)
    st = m.prepare(w, n_experts=E, top_k=k, max_tokens=T)
    data, _ = inputs.make_inputs("prefill" if T > 256 else "sweep", T, 3, cuda_dev)
    x, logits = data["hidden_states"], data["router_logits"]
    out, ids, tw = m.kernel_fn({"hidden_states": x, "router_logits": logits}, st, return_routing=True)
    torch.cuda.synchronize()
    assert m.read_status(st) == 0
    views = m.workspace_views(st, T)
    rid, _ = orc.route_topk(logits.cpu(), k)
    assert torch.equal(ids.cpu(), rid)
    sel = torch.arange(0, T, max(T // 8, 1))[:8]
    ref, parts, _ = _oracle_rows_of_tokens(orc, w, x, ids, tw, sel)
    assert _rel(out[sel.to(cuda_dev)], parts["out_fp32"]) <= TOL
    inv = views["inv"].cpu().view(T, k)
    rows_gpu = []
    for q in range(int(parts["off"][-1])):
        entry = int(parts["perm"][q])
        rows_gpu.append(int(inv[int(sel[entry // k]), entry % k]))
    rows_gpu = torch.tensor(rows_gpu, device=views["y"].device)
    assert _rel(views["inter"][rows_gpu], parts["inter"]) <= TOL
    assert _rel(views["y"][rows_gpu], parts["y"]) <= TOL


@pytest.mark.parametrize("T,tile", [(64, 16), (600, 128), (200, 64)])
def test_forward_expert_parallel_shape(cuda_dev, T, tile):
    """The per-expert shape of the expert-parallel configuration (H7168 I2048: 28 K stages for the
    gate/up GEMM, 8 for the down GEMM, 28 pairs of down tiles), four local experts of eight, top-4,
    with the narrow and the wide token tile."""
    m, inputs, _lib, orc = _mods()
    out, ref, parts, views, st, _ = _run_forward(m, inputs, orc, cuda_dev, 7168, 2048, 8, 4, T, seed=300 + T,
                                                 post_norm=True, lo=2, nloc=4, token_tile=tile)
    assert m.plan(st, T)[0] == tile
    _check_forward(out, ref, parts, views)


@pytest.mark.parametrize("tile", [0, 64, 16])
def test_forward_reference_skewed_counts(cuda_dev, tile):
    """The reference's own expert check (muse_prefill_layer/py/07_selftest.py:41-73): T = 700, counts
    [300, 200, 100, 60, 33, 17, 14, 5, 1] over nine experts, entries laid out as its
    `_routes_from_counts` does (entry idx of expert e's c-th row: token idx % T, slot idx // T; all
    other slots -1)."""
    m, inputs, _lib, orc = _mods()
    H, I, k, T = 1024, 512, 8, 700
    counts = [300, 200, 100, 60, 33, 17, 14, 5, 1]
    E = len(counts)
    ids = torch.full((T * k,), -1, dtype=torch.int32)
    r = 0
    for e, c in enumerate(counts):
        idx = torch.arange(r, r + c)
        ids[(idx % T) * k + idx // T] = e
        r += c
    ids = ids.view(T, k).to(cuda_dev)
    w = inputs.make_weights(H, I, E, 91, cuda_dev, post_norm=True)
    st = m.prepare(w, n_experts=E, top_k=k, max_tokens=T, token_tile=tile)
    g = torch.Generator(device=cuda_dev).manual_seed(17)
    x = torch.randn((T, H), generator=g, device=cuda_dev).to(torch.bfloat16)
    tw = torch.rand((T, k), generator=g, device=cuda_dev)
    out = m.kernel_fn({"hidden_states": x, "topk_ids": ids, "topk_weights": tw}, st)
    torch.cuda.synchronize()
    assert m.read_status(st) == 0
    ref, parts = orc.moe_forward(x, ids, tw, w, return_parts=True)
    assert parts["cnt"].tolist() == counts
    _check_forward(out, ref, parts, m.workspace_views(st, T))


SENTINEL = 0x5EADBEEF
GUARD_WORDS = 65536


def _guarded(t):
    """Copy of tensor t placed in front of 64 Ki sentinel words (the reference's guard scheme,
    muse_decode_layer/py/05_tune.py:453-477). Returns (view with t's shape and dtype, guard words)."""
    nbytes = t.numel() * t.element_size()
    pad = (nbytes + 255) // 256 * 256
    buf = torch.empty(pad + GUARD_WORDS * 4, dtype=torch.uint8, device=t.device)
    guard = buf[pad:].view(torch.int32)
    guard.fill_(SENTINEL)
    buf[nbytes:pad].view(torch.uint8).fill_(0xA5)
    view = buf[:nbytes].view(t.dtype).view(t.shape)
    view.copy_(t)
    return view, guard, buf[nbytes:pad]


def test_state_hygiene_token_sequence_and_guard_words(cuda_dev):
    """One state driven through the reference's token-count sequence 32, 16, 256, 8, 16, 128, 16
    (muse_decode_layer/py/17_moev.py:882-908): every output must equal, bit for bit, the output of a
    freshly prepared state on the same input (nothing a call leaves in the workspace may leak into the
    next), and 64 Ki sentinel words behind the output, the workspace and both packed weight buffers
    must survive every call."""
    m, inputs, _lib, orc = _mods()
    H, I, E, k, cap = 1024, 512, 16, 4, 256
    w = inputs.make_weights(H, I, E, 123, cuda_dev, post_norm=True)
    st = m.prepare(w, n_experts=E, top_k=k, max_tokens=cap)
    guards = []
    for key in ("workspace", "packed13", "packed2"):
        st[key], g, pad = _guarded(st[key])
        guards.append((key, g, pad))
    for step, T in enumerate((32, 16, 256, 8, 16, 128, 16)):
        g = torch.Generator(device=cuda_dev).manual_seed(500 + step)
        data = {"hidden_states": torch.randn((T, H), generator=g, device=cuda_dev).to(torch.bfloat16),
                "router_logits": torch.randn((T, E), generator=g, device=cuda_dev)}
        out_buf, out_guard, out_pad = _guarded(torch.empty((T, H), dtype=torch.bfloat16, device=cuda_dev))
        got = m.kernel_fn(data, st, out=out_buf)
        fresh = m.prepare(w, n_experts=E, top_k=k, max_tokens=cap)
        want = m.kernel_fn(data, fresh)
        torch.cuda.synchronize()
        assert torch.equal(got, want), (step, T)
        assert m.read_status(st) == 0 and m.read_status(fresh) == 0
        for key, gw, pad in guards + [("out", out_guard, out_pad)]:
            assert bool((gw == SENTINEL).all()), (step, T, key)
            assert bool((pad == 0xA5).all()), (step, T, key)
        if step == 0:   # and the first one against the oracle, so "equal" is not "equally wrong"
            _, ids, tw = m.kernel_fn(data, fresh, return_routing=True)
            ref = orc.moe_forward(data["hidden_states"], ids, tw, w).float()
            assert _rel(got, ref) <= TOL


def test_bounded_wait_runs_out_cleanly_and_the_state_recovers(cuda_dev):
    """Failure detection without a fault: the streaming probe is told to withhold one slot release, so
    its producer's bounded wait (one second) runs out; the kernel must come back by itself with the
    time-out status, leave the context usable, and the library must work normally afterwards. Then the
    recovery path of a state: a workspace whose control words were left dirty (as a kernel that gave
    up would leave them) is put back by reinit_workspace and gives the clean result again."""
    import time

    m, inputs, _lib, orc = _mods()
    t0 = time.time()
    gbs, status = m.bw_probe(nbytes=64 << 20, skip_release=2, device=cuda_dev)
    assert status == 1                       # MSK_DEV_ERR_TIMEOUT, reported, not trapped
    assert 0.5 < time.time() - t0 < 30.0     # the one-second limit, not an endless spin
    gbs, status = m.bw_probe(nbytes=256 << 20, device=cuda_dev)
    assert status == 0 and gbs > 500.0       # the context is alive and the same kernel streams again
    H, I, E, k, T = 1024, 512, 16, 4, 8
    w = inputs.make_weights(H, I, E, 7, cuda_dev, post_norm=True)
    st = m.prepare(w, n_experts=E, top_k=k, max_tokens=32, flat_shares=1, decode_path=1)
    g = torch.Generator(device=cuda_dev).manual_seed(3)
    data = {"hidden_states": torch.randn((T, H), generator=g, device=cuda_dev).to(torch.bfloat16),
            "router_logits": torch.randn((T, E), generator=g, device=cuda_dev)}
    clean = m.kernel_fn(data, st).clone()
    torch.cuda.synchronize()
    views = {}
    for which in (7, 8, 10):                 # unit tickets, control words of the few-token paths, tile hand-over counters
        ptr = ctypes.c_void_p()
        _lib.check(st["lib"].lib.msk_moe_workspace_view(ctypes.byref(st["cfg"]), _lib.ptr(st["workspace"]), which,
                                                        ctypes.byref(ptr)), "view")
        views[which] = ptr.value - st["workspace"].data_ptr()
    st["workspace"][views[7]:views[7] + 64].fill_(1)      # tickets half-way
    st["workspace"][views[8]:views[8] + 8192].fill_(3)    # token tickets, grid and tile counters
    st["workspace"][views[10]:views[10] + 64].fill_(5)    # gate/up units counted for tiles that no down unit took over
    st["workspace"][:4].copy_(torch.tensor([1, 0, 0, 0], dtype=torch.uint8))   # sticky status word
    assert m.read_status(st) == 1
    m.reinit_workspace(st)
    assert m.read_status(st) == 0
    for path in (1, 3):
        st["cfg"].decode_path = path
        got = m.kernel_fn(data, st)
        assert torch.equal(got, clean) if path == 1 else _rel(got, clean) <= 8e-3
        torch.cuda.synchronize()
        assert m.read_status(st) == 0


def test_state_dict_round_trip_skips_the_repack(cuda_dev):
    """state_dict() / load_state_dict(): the packed tiles, scales and configuration are enough to
    rebuild a state; kernel_fn on the rebuilt state gives the same bits."""
    import copy
    import io

    m, inputs, _lib, orc = _mods()
    H, I, E, k, T = 1024, 512, 8, 2, 40
    w = inputs.make_weights(H, I, E, 19, cuda_dev, post_norm=True)
    g = torch.Generator(device=cuda_dev).manual_seed(5)
    w["pre_norm_w"] = (torch.randn((H,), generator=g, device=cuda_dev) * 0.1).to(torch.bfloat16)
    w["router"] = torch.randn((E, H), generator=g, device=cuda_dev) * 0.02
    st = m.prepare(w, n_experts=E, top_k=k, max_tokens=64, routing_mode="softmax_topk")
    x = torch.randn((T, H), generator=g, device=cuda_dev).to(torch.bfloat16)
    want = m.kernel_fn({"hidden_states": x}, st)
    buf = io.BytesIO()
    torch.save(m.state_dict(st), buf)
    buf.seek(0)
    st2 = m.load_state_dict(torch.load(buf, map_location="cpu"), device=cuda_dev)
    assert st2["cfg"].hidden == H and st2["cfg"].max_tokens == 64
    assert torch.equal(m.kernel_fn({"hidden_states": x}, st2), want)
    assert torch.equal(m.kernel_fn({"hidden_states": x}, copy.deepcopy(st2)), want)
    back = m.export_weights(st2)
    assert torch.equal(back["w13"], w["w13"]) and torch.equal(back["w2_sf"], w["w2_sf"].view(torch.uint8))


def test_prefill_moe_runs_the_prefill_layer_call_site(cuda_dev):
    """The prefill layer's expert step (muse_prefill_layer/py/04_moe_forward.py:6-52 followed by its
    combine): un-normed pooler rows, local ids with -1, routing weights in; pre-expert norm, both
    GEMMs, post-expert norm and weighted sum out. T = 700 with the reference's skewed counts."""
    m, inputs, _lib, orc = _mods()
    from muse_moe_w4a16.compat import PrefillMoe

    H, I, k, T = 1024, 512, 8, 700
    counts = [300, 200, 100, 60, 33, 17, 14, 5, 1]
    E = len(counts)
    lid = torch.full((T * k,), -1, dtype=torch.int32)
    pos = torch.zeros((T * k,), dtype=torch.int32)
    r = 0
    for e, c in enumerate(counts):
        idx = torch.arange(r, r + c)
        lid[(idx % T) * k + idx // T] = e
        pos[(idx % T) * k + idx // T] = torch.arange(c, dtype=torch.int32)
        r += c
    lid, pos = lid.view(T, k).to(cuda_dev), pos.view(T, k).to(cuda_dev)
    cnt = torch.tensor(counts, dtype=torch.int32, device=cuda_dev)
    w = inputs.make_weights(H, I, E, 23, cuda_dev, post_norm=True)
    g = torch.Generator(device=cuda_dev).manual_seed(29)
    w["pre_norm_w"] = (torch.randn((H,), generator=g, device=cuda_dev) * 0.1).to(torch.bfloat16)
    ext = PrefillMoe(m.prepare(w, local_start=0, n_experts=E, top_k=k, max_tokens=T))
    p = (torch.randn((T, H), generator=g, device=cuda_dev) * 2.0).to(torch.bfloat16)
    topw = torch.rand((T, k), generator=g, device=cuda_dev)
    moe_out = torch.full((T, H), float("nan"), dtype=torch.bfloat16, device=cuda_dev)
    ex = ext.moe_forward(p, lid, pos, cnt, T, topw, out=moe_out)
    ext.moe_combine(None, ex["rrow"], lid, topw, w["post_norm_w"], moe_out)
    torch.cuda.synchronize()
    ref, parts = orc.moe_forward(p, lid, topw, w, return_parts=True)
    assert _rel(moe_out, parts["out_fp32"]) <= TOL
    assert ex["out"].data_ptr() == moe_out.data_ptr()
    assert np.array_equal(ex["rrow"].tensor().cpu().numpy().reshape(-1), parts["inv"])


def test_activations_outside_the_f16_range_saturate_as_documented(cuda_dev):
    """The MMA operands are F16: a BF16 activation beyond +-65504 enters the GEMM as +-65504 (and one
    below 2^-24 as zero), and so does a SwiGLU value that large. The result must equal the oracle
    evaluated with its operands saturated the same way, and rows inside the range must not be affected
    by a saturating neighbour."""
    m, inputs, _lib, orc = _mods()
    H, I, E, k, T = 512, 256, 8, 2, 6
    w = inputs.make_weights(H, I, E, 31, cuda_dev)
    st = m.prepare(w, n_experts=E, top_k=k, max_tokens=T)
    g = torch.Generator(device=cuda_dev).manual_seed(37)
    x = torch.randn((T, H), generator=g, device=cuda_dev).to(torch.bfloat16)
    x[1, 5] = 3.0e5          # beyond the F16 range
    x[1, 9] = -1.0e6
    x[2, 7] = 1.0e-9         # below the smallest F16 subnormal
    logits = torch.randn((T, E), generator=g, device=cuda_dev)
    out, ids, tw = m.kernel_fn({"hidden_states": x, "router_logits": logits}, st, return_routing=True)
    torch.cuda.synchronize()
    ref = orc.moe_forward(x, ids, tw, w, f16_operands=True).float()   # x and inter saturated as the F16 operands are
    assert torch.isfinite(out.float()).all()
    assert _rel(out, ref) <= TOL
    plain = orc.moe_forward(x, ids, tw, w).float()
    keep = [0, 2, 3, 4, 5]
    assert _rel(out[keep], plain[keep]) <= TOL


@pytest.mark.parametrize("T,E,H", [(16, 128, 512), (50, 256, 1024), (300, 8, 512), (1000, 128, 4096), (130, 384, 2048)])
def test_router_logits_gemm_on_the_hi_lo_pair(cuda_dev, T, E, H):
    """msk_moe_router_logits_hilo: the FP32 router weight as the reference's exact-sum BF16 pair
    (muse_decode_layer/py/05_tune.py:279-286) through the tensor-core GEMM. The logits must equal the
    FP64 product of x with hi + lo up to FP32 accumulation, stay within what w - hi - lo drops of the
    FP32 product, repeat bit for bit, and give the FP32 matvec's top-k except where two scores are
    closer than that difference (reported as tie-risk, not as a failure)."""
    m, inputs, _lib, orc = _mods()
    lib = _lib.load()
    g = torch.Generator(device=cuda_dev).manual_seed(T + E)
    w = torch.randn((E, H), generator=g, device=cuda_dev) * 0.02
    x = torch.randn((T, H), generator=g, device=cuda_dev).to(torch.bfloat16)
    hilo = m.split_router(w)
    assert hilo.dtype == torch.bfloat16 and tuple(hilo.shape) == (2 * E, H)
    k = min(8, E)
    cfg = _lib.MskMoeCfg(hidden=H, inter=256, n_experts=E, local_start=0, local_count=min(E, 256), top_k=k, max_tokens=T)
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    status = torch.zeros(4, dtype=torch.int32, device=cuda_dev)

    def gemm():
        out = torch.full((T, E), float("nan"), device=cuda_dev)
        _lib.check(lib.msk_moe_router_logits_hilo(ctypes.byref(cfg), _lib.ptr(x), _lib.ptr(hilo), _lib.ptr(out),
                                                  _lib.ptr(status), T, st), "router_logits_hilo")
        return out

    a = gemm()
    b = gemm()
    mv = torch.empty((T, E), device=cuda_dev)
    _lib.check(lib.msk_moe_router_logits(ctypes.byref(cfg), _lib.ptr(x), _lib.ptr(w), _lib.ptr(mv), T, st), "router_logits")
    torch.cuda.synchronize()
    assert int(status[0]) == 0 and torch.equal(a, b) and torch.isfinite(a).all()
    xd = x.double()
    pair = xd @ (hilo[:E].double() + hilo[E:].double()).T
    full = xd @ w.double().T
    scale = float(full.abs().max())
    assert float((a.double() - pair).abs().max()) <= 2e-5 * scale      # FP32 accumulation of exact products (up to 8192 of them)
    assert float((a.double() - full).abs().max()) <= 5e-5 * scale      # plus the part of w the pair drops
    ia, _ = orc.route_topk(a.cpu(), k)
    ib, _ = orc.route_topk(mv.cpu(), k)
    rows, slots = np.nonzero(ia.numpy() != ib.numpy())
    fl = full.cpu().numpy()
    for r, c in zip(rows, slots):      # tie-risk: the two candidates' exact scores are closer than the logits' error
        assert abs(fl[r, ia[r, c]] - fl[r, ib[r, c]]) <= 1e-4 * scale, (r, c)
    assert len(set(rows.tolist())) <= max(1, T // 50)


def test_kernel_fn_with_router_weight_uses_the_gemm_from_sixteen_tokens(cuda_dev):
    """weights["router"]: few tokens take the FP32 matvec, 16 and more the hi + lo GEMM; both feed the
    same routing and expert kernels, and the output matches the oracle on the routing the module used."""
    m, inputs, _lib, orc = _mods()
    H, I, E, k = 1024, 512, 16, 4
    w = inputs.make_weights(H, I, E, 41, cuda_dev)
    g = torch.Generator(device=cuda_dev).manual_seed(43)
    w["router"] = torch.randn((E, H), generator=g, device=cuda_dev) * 0.02
    st = m.prepare(w, n_experts=E, top_k=k, max_tokens=256)
    for T in (5, 16, 200):
        x = torch.randn((T, H), generator=g, device=cuda_dev).to(torch.bfloat16)
        out, ids, tw = m.kernel_fn({"hidden_states": x}, st, return_routing=True)
        torch.cuda.synchronize()
        assert m.read_status(st) == 0
        rid, _ = orc.route_topk(orc.router_logits(x.cpu(), w["router"].cpu()), k)
        assert float((ids.cpu() == rid).all(dim=1).float().mean()) >= 0.97      # near-ties may pick the neighbour
        ref = orc.moe_forward(x, ids, tw, w).float()
        assert _rel(out, ref) <= TOL
