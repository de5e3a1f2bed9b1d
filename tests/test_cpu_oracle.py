"""CPU tests: the oracle against the reference-generated golden vectors and hand-computed
known answers, the quantiser, and the host side of the C ABI (no GPU, no compute calls)."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

from oracle import moe_oracle as orc

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
GOLD = np.load(os.path.join(HERE, "golden", "reference_vectors.npz"))


# ------------------------------------------------------------ golden vectors
def test_nibble_order_matches_reference_split_nibbles():
    codes, rows = GOLD["nib_codes"], GOLD["nib_rows"]
    assert np.array_equal(orc.split_nibbles(codes[rows]), GOLD["nib_out"])


def test_e4m3_table_matches_reference_lut():
    lut = GOLD["e4m3_lut"].astype(np.int64) & 0xFFFF           # bf16 bits of value * 2^64
    vals = orc.e4m3_value(np.arange(256, dtype=np.uint8))
    want = torch.from_numpy(lut.astype(np.int16)).view(torch.bfloat16).float().numpy()
    nan = np.isnan(vals)
    assert list(np.nonzero(nan)[0]) == [0x7F, 0xFF]
    assert np.array_equal(np.isnan(want), nan)
    assert np.array_equal(vals[~nan].astype(np.float64) * 2.0 ** 64, want[~nan].astype(np.float64))


@pytest.mark.parametrize("bs", [4, 33])
def test_sort_on_reference_generated_routing(bs):
    ids = GOLD[f"gen{bs}_ids"]
    w = GOLD[f"gen{bs}_w"]
    assert ids.shape == (bs, 8) and np.allclose(w.sum(-1), 1.0, atol=1e-5)
    cnt, off, perm, inv = orc.sort_routes(ids, 0, 32)  # the reference rank owns experts 0..31
    flat = ids.reshape(-1)
    local = (flat >= 0) & (flat < 32)
    assert cnt.sum() == local.sum() == off[-1]
    # same answer as a stable sort of the local ids (the bit-exactness target of the kernel)
    lid = torch.from_numpy(np.where(local, flat, 1 << 20))
    order = torch.sort(lid, stable=True).indices.numpy()[: int(off[-1])]
    assert np.array_equal(perm, order)
    assert np.array_equal(inv[perm], np.arange(len(perm)))
    assert np.all(inv[~local] == -1)
    for e in range(32):
        seg = perm[off[e]:off[e + 1]]
        assert np.all(flat[seg] == e) and np.all(np.diff(seg) > 0)


# --------------------------------------------------------- known-answer tests
def test_e2m1_codes_known_answers():
    want = [0, .5, 1, 1.5, 2, 3, 4, 6, -0.0, -.5, -1, -1.5, -2, -3, -4, -6]
    got = orc.e2m1_value(np.arange(16, dtype=np.uint8))
    assert np.array_equal(got, np.array(want, dtype=np.float32))
    assert np.signbit(got[8])


@pytest.mark.parametrize("byte,value", [(0x00, 0.0), (0x01, 2.0 ** -9), (0x07, 7 * 2.0 ** -9), (0x08, 2.0 ** -6),
                                        (0x38, 1.0), (0x40, 2.0), (0x7E, 448.0), (0xB8, -1.0)])
def test_e4m3_known_answers(byte, value):
    assert float(orc.e4m3_value(np.uint8(byte))) == value


def test_dequant_known_answers_all_codes_times_scales():
    scales = [0x00, 0x01, 0x07, 0x08, 0x38, 0x40, 0x7E]
    sv = [0.0, 2.0 ** -9, 7 * 2.0 ** -9, 2.0 ** -6, 1.0, 2.0, 448.0]
    e2 = [0, .5, 1, 1.5, 2, 3, 4, 6]
    codes = np.array([[(2 * j) | ((2 * j + 1) << 4) for j in range(8)]] * len(scales), dtype=np.uint8)  # k = 0..15
    sf = np.array([[s] for s in scales], dtype=np.uint8)
    for gs in (1.0, 3.0e-5):
        got = orc.dequant(codes, sf, gs)
        for r, s in enumerate(sv):
            for k in range(16):
                want = np.float32((-1 if k >= 8 else 1) * e2[k % 8] * s) * np.float32(gs)
                assert got[r, k] == want


def test_quantiser_round_trip_and_tie_rule():
    from muse_moe_w4a16 import quant

    ties = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -0.25, -5.0, 7.0, 0.0])
    codes = quant.e2m1_codes(ties)
    assert codes.tolist() == [0, 2, 2, 4, 4, 6, 6, 8, 14, 7, 0]  # ties go to the even code
    g = torch.Generator().manual_seed(0)
    w = (torch.randn((64, 256), generator=g) * 0.02).to(torch.bfloat16)
    c, s, gs = quant.quantize_nvfp4(w)
    assert c.shape == (64, 128) and s.shape == (64, 16)
    assert abs(float(gs) - float(w.float().abs().max()) / (6 * 448)) < 1e-12
    dq = orc.dequant(c.numpy(), s.numpy(), float(gs))
    blk = w.float().view(64, 16, 16).abs().amax(-1).numpy().repeat(16, -1).reshape(64, 256)
    assert np.all(np.abs(dq - w.float().numpy()) <= 0.26 * blk + 1e-12)  # half an E2M1 step at the block top
    assert 0x08 <= int(s.min()) and int(s.max()) <= 0x7E                  # normal scale bytes only (neither zero, subnormal nor NaN)


def test_route_topk_tie_rule_and_weights():
    logits = torch.tensor([[1.0, 3.0, 3.0, -1.0, 3.0, 0.5]])
    ids, w = orc.route_topk(logits, 3)
    assert ids.tolist() == [[1, 2, 4]]
    assert torch.allclose(w, torch.full((1, 3), 1 / 3))
    ids, w = orc.route_topk(logits, 2, "sigmoid_bias", bias=torch.tensor([0, 0, 0, 5.0, 0, 0]), scale=1.0)
    assert ids.tolist() == [[3, 1]]
    s = torch.sigmoid(torch.tensor([-1.0, 3.0]))
    assert torch.allclose(w[0], s / s.sum())


def test_moe_forward_against_dense_evaluation():
    """The grouped oracle equals a dense per-token evaluation of the same formula."""
    from muse_moe_w4a16 import inputs

    H, I, E, k, T = 256, 256, 4, 2, 6
    w = inputs.make_weights(H, I, E, 1, "cpu", post_norm=True)
    g = torch.Generator().manual_seed(2)
    x = torch.randn((T, H), generator=g).to(torch.bfloat16)
    ids, tw = orc.route_topk(torch.randn((T, E), generator=g), k)
    out, parts = orc.moe_forward(x, ids, tw, w, return_parts=True)
    ref = torch.zeros((T, H))
    for t in range(T):
        for s in range(k):
            e = int(ids[t, s])
            y = orc.expert_forward(x[t:t + 1], w["w13"][e], w["w13_sf"][e], w["w13_gs"][e], w["w2"][e], w["w2_sf"][e],
                                   w["w2_gs"][e])[0]
            y = y * (1 + w["post_norm_w"].float())
            y = y * torch.rsqrt(y.pow(2).mean() + 1e-8)
            ref[t] += tw[t, s] * y
    assert torch.allclose(parts["out_fp32"], ref, rtol=1e-5, atol=1e-6)
    # local-range filter: the two halves of the experts sum to the whole (partial sums, EP "filter" mode)
    lo = {key: (v[:2] if key != "post_norm_w" else v) for key, v in w.items()}
    hi = {key: (v[2:] if key != "post_norm_w" else v) for key, v in w.items()}
    _, p0 = orc.moe_forward(x, ids, tw, lo, local_start=0, return_parts=True)
    _, p1 = orc.moe_forward(x, ids, tw, hi, local_start=2, return_parts=True)
    assert torch.allclose(p0["out_fp32"] + p1["out_fp32"], parts["out_fp32"], rtol=1e-5, atol=1e-6)


# ------------------------------------------------------------ C ABI, host side
def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "msk_moe.h")).read()
    return sorted(set(re.findall(r"^int (msk_\w+)\(", text, flags=re.M)))


def test_library_exports_every_declared_symbol():
    from muse_moe_w4a16 import _lib

    lib = _lib.load()
    declared = _declared_symbols()
    assert len(declared) >= 14
    for name in declared:
        assert hasattr(lib, name), name
    assert sorted(_lib.SIGNATURES) == declared  # the binding table and the header agree


def test_host_side_validation_rejects_bad_arguments():
    from muse_moe_w4a16 import _lib

    lib = _lib.load()
    good = dict(hidden=512, inter=256, n_experts=8, local_start=0, local_count=8, top_k=2, max_tokens=4)
    cfg = _lib.MskMoeCfg(**good)
    a, b = ctypes.c_size_t(), ctypes.c_size_t()
    assert lib.msk_moe_packed_bytes(ctypes.byref(cfg), ctypes.byref(a), ctypes.byref(b)) == 0
    assert a.value == 8 * (2 * 256 // 128) * (512 // 256) * 18432 and b.value == 8 * (512 // 128) * 1 * 18432
    assert lib.msk_moe_packed_bytes(None, ctypes.byref(a), ctypes.byref(b)) == -1
    for bad in (dict(hidden=500), dict(inter=128), dict(top_k=0), dict(top_k=17), dict(local_count=0),
                dict(local_count=300), dict(n_experts=600), dict(token_tile=8), dict(token_tile=48),
                dict(decode_path=5), dict(decode_path=-1)):
        c = _lib.MskMoeCfg(**{**good, **bad})
        assert lib.msk_moe_packed_bytes(ctypes.byref(c), ctypes.byref(a), ctypes.byref(b)) == -2, bad
    c = _lib.MskMoeCfg(**{**good, "local_start": 4})
    assert lib.msk_moe_packed_bytes(ctypes.byref(c), ctypes.byref(a), ctypes.byref(b)) == -5
    ws = ctypes.c_size_t()
    assert lib.msk_moe_workspace_bytes(ctypes.byref(cfg), ctypes.byref(ws)) == 0 and ws.value > 4 * 2 * 512 * 4
    # forward: NULL pointers, too many tokens, undersized workspace are refused before any launch
    p = ctypes.c_void_p(0)
    assert lib.msk_moe_forward(ctypes.byref(cfg), p, p, p, p, p, p, p, p, p, p, 0, 1, p) == -1
    fake = ctypes.c_void_p(4096)
    assert lib.msk_moe_forward(ctypes.byref(cfg), fake, fake, fake, fake, None, fake, fake, fake, fake, fake,
                               ws.value, 5, None) == -6
    assert lib.msk_moe_forward(ctypes.byref(cfg), fake, fake, fake, fake, None, fake, fake, fake, fake, fake,
                               16, 4, None) == -4
    odd = ctypes.c_void_p(4100)
    assert lib.msk_moe_forward(ctypes.byref(cfg), odd, fake, fake, fake, None, fake, fake, fake, fake, fake,
                               ws.value, 4, None) == -3
    plan = (ctypes.c_int * 4)()
    assert lib.msk_moe_plan(ctypes.byref(cfg), 4, plan) == 0 and plan[0] in (16, 32, 64, 128)


def _pieces(lib, n_base, nst, shares, mode, cta, heavy=0, skip=0):
    cap = 4096
    buf = (ctypes.c_int * (6 * cap))()
    n = ctypes.c_int()
    assert lib.msk_moe_share_pieces(n_base, nst, shares, mode, cta, heavy, skip, buf, cap, ctypes.byref(n)) == 0
    return [tuple(buf[6 * i:6 * i + 6]) for i in range(n.value)]


@pytest.mark.parametrize("n_base,nst,shares", [(96, 16, 148), (128, 6, 148), (600, 16, 148), (3, 28, 148), (1, 1, 7),
                                               (0, 16, 148), (37, 5, 5), (224, 8, 148), (50, 2, 1)])
def test_flat_shares_cover_every_stage_once_and_name_their_pieces(n_base, nst, shares):
    """The work distribution of the GEMM kernels (host twin of the device code): with flat shares (full
    rounds of whole units, then the last full round and the left-over units cut into equal shares of
    stages; nothing is cut when there are fewer units than CTAs)
    every (unit, stage) item belongs to exactly one CTA, shares differ by at most one item, a cut unit's
    pieces sit in consecutive CTAs in ascending K order, each in a slot of its own, and the first / last
    owner every piece computes is the CTA that really holds the unit's first / last stage."""
    from muse_moe_w4a16 import _lib

    lib = _lib.load()
    seen = {}
    sizes = []
    slots = set()
    for c in range(shares):
        pcs = _pieces(lib, n_base, nst, shares, 1, c)
        sizes.append(sum(k1 - k0 for _, k0, k1, *_ in pcs))
        for base, k0, k1, slot, first, last in pcs:
            assert 0 <= k0 < k1 <= nst
            for ks in range(k0, k1):
                assert (base, ks) not in seen
                seen[(base, ks)] = c
            if slot >= 0:
                assert slot not in slots and slot // 2 == c
                slots.add(slot)
            else:
                assert (k0, k1) == (0, nst)
    assert len(seen) == n_base * nst
    if n_base >= shares:
        assert max(sizes) - min(sizes) <= 1
    else:                       # fewer units than CTAs: nothing is cut
        assert set(sizes) <= {0, nst} and not slots
    for c in range(shares):
        for base, k0, k1, slot, first, last in _pieces(lib, n_base, nst, shares, 1, c):
            assert first == seen[(base, 0)] and last == seen[(base, nst - 1)]
            owners = [seen[(base, ks)] for ks in range(nst)]
            assert owners == sorted(owners) and first <= min(owners) and max(owners) <= last
            # every share between the first and the last owner either holds a piece of the unit or has an empty
            # share of the tail (the units left over after the full rounds of whole units)
            tail_first = n_base if n_base < shares else (n_base // shares - 1) * shares
            tail_items = (n_base - tail_first) * nst
            empty = lambda c: tail_items * (c + 1) // shares == tail_items * c // shares
            assert all(c in owners or empty(c) for c in range(first, last + 1))


def test_whole_unit_mode_gives_every_unit_to_one_cta():
    from muse_moe_w4a16 import _lib

    lib = _lib.load()
    n_base, nst, shares = 301, 16, 148
    got = []
    for c in range(shares):
        for base, k0, k1, slot, first, last in _pieces(lib, n_base, nst, shares, 0, c):
            assert (k0, k1, slot) == (0, nst, -1)
            got.append(base)
    assert sorted(got) == list(range(n_base))


@pytest.mark.parametrize("n0,nst0,n1,nst1,shares", [(600, 16, 800, 6, 148), (96, 16, 128, 6, 148), (1356, 16, 1808, 6, 148),
                                                     (300, 28, 100, 8, 148), (5, 2, 3, 1, 4)])
def test_skewed_dealing_of_the_second_phase_balances_both_phases(n0, nst0, n1, nst1, shares):
    """One launch for both GEMMs: the CTAs that hold one more gate/up unit are left out of the first
    rounds of down units. Every down unit still goes to exactly one CTA, each CTA takes its units in
    ascending order, and the largest total (in K stages) is no larger than with plain round-robin."""
    from muse_moe_w4a16 import _lib

    lib = _lib.load()
    heavy = n0 % shares if n0 >= shares else 0   # the rule of the kernel (phase1_skew)
    skip = (nst0 + nst1 // 2) // nst1 if heavy else 0
    load0 = [len(_pieces(lib, n0, nst0, shares, 0, c)) * nst0 for c in range(shares)]
    got, skewed, plain = [], [], []
    for c in range(shares):
        mine = [b for b, *_ in _pieces(lib, n1, nst1, shares, 0, c, heavy, skip)]
        assert mine == sorted(mine)
        got += mine
        skewed.append(load0[c] + len(mine) * nst1)
        plain.append(load0[c] + len(_pieces(lib, n1, nst1, shares, 0, c)) * nst1)
    assert sorted(got) == list(range(n1))
    assert max(skewed) <= max(plain)


def test_plan_is_a_function_of_the_configuration_only():
    """Token tile, path and grid follow from the shapes and the token count (never from the device:
    the default grid is a constant): up to 8 tokens the whole step is one launch, beyond that the narrow
    token tiles run both GEMMs in one launch behind the sort (path 4), the wide tiles the chain."""
    from muse_moe_w4a16 import _lib

    lib = _lib.load()
    plan = (ctypes.c_int * 4)()
    cfg = _lib.MskMoeCfg(hidden=4096, inter=1536, n_experts=128, local_start=0, local_count=128, top_k=8, max_tokens=8192)
    want = {1: (16, 0, 0, 148), 8: (16, 0, 0, 148), 9: (16, 4, 0, 148), 32: (16, 4, 0, 148), 64: (16, 4, 0, 148),
            256: (64, 1, 0, 148), 8192: (128, 1, 0, 148)}
    for T, w in want.items():
        assert lib.msk_moe_plan(ctypes.byref(cfg), T, plan) == 0
        assert tuple(plan) == w, (T, tuple(plan))
    cfg.decode_path = 2
    cfg.flat_shares = 1
    assert lib.msk_moe_plan(ctypes.byref(cfg), 8, plan) == 0 and tuple(plan) == (16, 2, 1, 148)
    cfg.decode_path = 3
    assert lib.msk_moe_plan(ctypes.byref(cfg), 32, plan) == 0 and tuple(plan) == (16, 0, 0, 148)
    cfg.decode_path = 4
    assert lib.msk_moe_plan(ctypes.byref(cfg), 190, plan) == 0 and tuple(plan) == (16, 4, 0, 148)
    cfg.token_tile = 32
    assert lib.msk_moe_plan(ctypes.byref(cfg), 190, plan) == 0 and tuple(plan) == (32, 4, 0, 148)
    cfg.token_tile = 0
    assert lib.msk_moe_plan(ctypes.byref(cfg), 256, plan) == 0 and tuple(plan) == (64, 1, 0, 148)   # wide tile: the chain
    cfg.decode_path = 1
    cfg.num_ctas = 37
    assert lib.msk_moe_plan(ctypes.byref(cfg), 8, plan) == 0 and tuple(plan) == (16, 1, 1, 37)
    assert lib.msk_moe_plan(ctypes.byref(cfg), 64, plan) == 0 and tuple(plan) == (16, 1, 0, 37)


def test_workspace_init_covers_every_control_word():
    """msk_moe_workspace_init zeroes everything in front of `inter`: the status word, the sort tables,
    both ticket regions, the control words of the few-token paths (token tickets, grid and tile
    counters), the per-CTA counts of the multi-CTA sort and the tile counters of the hand-over between the
    two GEMM launches must all lie there."""
    from muse_moe_w4a16 import _lib

    lib = _lib.load()
    cfg = _lib.MskMoeCfg(hidden=4096, inter=1536, n_experts=128, local_start=0, local_count=128, top_k=8, max_tokens=256)
    base = 1 << 20

    def off(which):
        p = ctypes.c_void_p()
        assert lib.msk_moe_workspace_view(ctypes.byref(cfg), ctypes.c_void_p(base), which, ctypes.byref(p)) == 0
        return p.value - base

    inter = off(4)
    pairs = max(1536 // 128, 4096 // 256)
    tiles = 256 * 8 // 16 + 128
    for which, nbytes in ((0, 128 * 4), (1, 129 * 4), (2, 2048 * 4), (3, 2048 * 4), (7, 2 * tiles * pairs * 4),
                          (8, 8192), (9, 64 * 256 * 4), (10, 2 * tiles * 4)):
        assert 256 <= off(which) and off(which) + nbytes <= inter, which
    ws = ctypes.c_size_t()
    assert lib.msk_moe_workspace_bytes(ctypes.byref(cfg), ctypes.byref(ws)) == 0
    assert ws.value < 200 << 20      # the pieces of cut units take two slots per CTA, not a split-K buffer per unit


def test_module_refuses_cpu_tensors():
    import muse_moe_w4a16 as moe
    from muse_moe_w4a16 import inputs

    w = inputs.make_weights(256, 256, 2, 0, "cpu")
    with pytest.raises(RuntimeError, match="CUDA"):
        moe.prepare(w)


def test_oracle_pre_expert_norm_is_the_norm_in_front_of_the_step():
    """pre_expert_norm follows muse_decode_layer/py/04_triton_kernels.py:556-568 (RMS over the row,
    eps 1e-5, times 1 + g, one rounding to bf16), and moe_forward with weights["pre_norm_w"] equals
    moe_forward on the normed rows."""
    from muse_moe_w4a16 import inputs
    from oracle import moe_oracle as orc

    H, I, E, k, T = 256, 256, 4, 2, 5
    w = inputs.make_weights(H, I, E, 3, "cpu", post_norm=True)
    g = torch.Generator().manual_seed(2)
    x = (torch.randn((T, H), generator=g) * 2.0).to(torch.bfloat16)
    gw = (torch.randn((H,), generator=g) * 0.1).to(torch.bfloat16)
    xn = orc.pre_expert_norm(x, gw)
    xf = x.float()
    want = xf / torch.sqrt((xf * xf).sum(-1, keepdim=True) / H + 1e-5) * (1.0 + gw.float())
    assert xn.dtype == torch.bfloat16
    assert float((xn.float() - want).abs().max()) <= 2.0 ** -8 * float(want.abs().max())
    ids, tw = orc.route_topk(torch.randn((T, E), generator=g), k)
    a = orc.moe_forward(x, ids, tw, dict(w, pre_norm_w=gw))
    b = orc.moe_forward(xn, ids, tw, w)
    assert torch.equal(a, b)


# ------------------------------- vectors produced by the reference's Triton kernels on a CPU
def _bf16(a):
    return torch.from_numpy(a.astype(np.int16)).view(torch.bfloat16)


def test_routing_matches_reference_route_split():
    """ids, local ids and weights of the reference's `_route_split` (sigmoid(logit / sqrt(32)) + bias,
    eight rounds of arg-max, ties to the lowest index), on logits that hold exact ties."""
    logits, bias = torch.from_numpy(GOLD["rs_logits"]), torch.from_numpy(GOLD["rs_bias"])
    ids, w = orc.route_topk(logits, 8, "sigmoid_bias", bias)
    assert np.array_equal(ids.numpy(), GOLD["rs_ids"])
    assert np.allclose(w.numpy(), GOLD["rs_w"], rtol=2e-6, atol=1e-8)
    # the constructed ties are there and went to the lower index
    assert list(GOLD["rs_ids"][1]) == sorted(GOLD["rs_ids"][1].tolist(), key=lambda e: (-float(bias[e]), e))
    assert not np.isin(GOLD["rs_ids"], np.arange(200, 208)).any() or np.isin(GOLD["rs_ids"], np.arange(8, 16)).any()
    ls = int(GOLD["rs_local_start"][0])
    assert np.array_equal(orc.local_ids(ids, ls, 32).numpy(), GOLD["rs_lids"])
    # the stable sort drops exactly the entries the reference marks -1
    cnt, off, perm, inv = orc.sort_routes(GOLD["rs_ids"], ls, 32)
    assert np.array_equal(inv >= 0, GOLD["rs_lids"].reshape(-1) >= 0)
    assert np.array_equal(GOLD["rs_lids"].reshape(-1)[perm], np.sort(GOLD["rs_lids"].reshape(-1)[perm], kind="stable"))


def _trunc_bf16(f):
    """FP32 -> BF16 by dropping the low 16 bits: how Triton's CPU interpreter converts (compiled for
    a GPU the same kernels round to nearest even, as the oracle and the CUDA path do). The golden
    BF16 outputs are therefore compared with the truncated FP32 values of the oracle, which pins the
    FP32 arithmetic in front of the rounding."""
    return (f.contiguous().view(torch.int32) & -65536).view(torch.float32)


def test_pre_expert_norm_matches_reference_route_split():
    """The expert input the reference's routing kernel stores: x * rsqrt(sum(x^2)/H + 1e-5) * (1 + g)."""
    f = orc.pre_expert_norm(_bf16(GOLD["rs_pooled"]), _bf16(GOLD["rs_gpre"]), return_fp32=True)
    want = _bf16(GOLD["rs_x"]).float()
    same = _trunc_bf16(f) == want
    # a row's sum of 4096 squares is taken in another order by the two programs: allow the last FP32 bit
    # of the scale to move a value across a BF16 boundary on a handful of elements
    assert float(same.float().mean()) > 0.999
    assert bool(((f - want).abs() <= 2.0 ** -7 * want.abs() + 1e-30).all())
    rn = orc.pre_expert_norm(_bf16(GOLD["rs_pooled"]), _bf16(GOLD["rs_gpre"]))
    assert rn.dtype == torch.bfloat16 and bool(((rn.float() - f).abs() <= 2.0 ** -8 * f.abs()).all())


def test_combine_matches_reference_pexp_norm_sum():
    """Post-expert norm (1 + w first, RMS over the row, eps 1e-8) times the routing weight, summed in
    slot order over the slots with a local expert; a token without one is zero."""
    y = _bf16(GOLD["pn_y"]).float()
    pw = _bf16(GOLD["pn_w"]).float()
    s, lid = torch.from_numpy(GOLD["pn_s"]), torch.from_numpy(GOLD["pn_ids"])
    T, K = lid.shape
    inv = torch.where(lid >= 0, torch.arange(T * K, dtype=torch.int32).view(T, K), torch.full_like(lid, -1))
    out = orc.combine_rows(y * (1.0 + pw), inv, s, True, 1e-8)
    want = _bf16(GOLD["pn_out"]).float()
    assert float(want[2].abs().max()) == 0.0 and float(out[2].abs().max()) == 0.0
    same = _trunc_bf16(out) == want
    assert float(same.float().mean()) > 0.995          # the rest straddle a BF16 boundary in their last FP32 bits
    assert float((out - want).abs().max()) <= 2.0 ** -7 * float(want.abs().max())


def test_timeline_stamp_slots_follow_the_kernel_enum():
    """muse_moe_w4a16.timeline names the kernels' trace slots by number; the numbers must be the positions
    of the TR_* enumerators in csrc/gemm.cuh."""
    import re

    from muse_moe_w4a16 import timeline

    src = open(os.path.join(ROOT, "muse-spark-kernels_b200", "csrc", "gemm.cuh")).read()
    body = re.search(r"enum\s*:\s*int\s*\{\s*(TR_START\s*=\s*0.*?)\};", src, re.S).group(1)
    names = [n.strip().split("=")[0].strip() for n in body.replace("\n", " ").split(",") if n.strip()]
    slots = {n[3:]: i for i, n in enumerate(names)}
    assert len(slots) <= 16                      # 16 stamps per CTA in the workspace
    for name, slot in timeline.STAMPS:
        assert slots[name] == slot, name
    assert {n for n, _ in timeline.STAMPS} == set(slots)
