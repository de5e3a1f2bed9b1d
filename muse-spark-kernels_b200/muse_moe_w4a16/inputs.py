"""Seeded synthetic inputs with the shapes and distributions of the benchmark configs.

They stand in for the benchmark harness's input generator, which the reference only
restates (muse_moe_w4a16/py/04_diag.py:6-21). Everything comes from torch.Generator(seed).
"""
import math

import torch

from .quant import random_nvfp4_experts

# name -> (H, I, E, top_k, router kind)
SHAPES = {
    "tiny": dict(H=512, I=256, E=8, k=2, router="weight"),         # config 0 (T=4)
    "decode": dict(H=4096, I=1536, E=128, k=8, router="uniform"),  # config 1 (T=1)
    "sweep": dict(H=4096, I=1536, E=128, k=8, router="normal"),    # config 2 (T in 1..256)
    "prefill": dict(H=4096, I=1536, E=128, k=8, router="zipf"),    # config 3 (T=8192)
    "ep": dict(H=7168, I=2048, E=256, k=8, router="uniform"),      # config 4 (T=4096 per GPU)
}


def make_weights(H, I, n_local, seed, device, post_norm=False):
    """The reference's `Weights` dict (muse_moe_w4a16/py/00_moe_w4a16.py:72-80) for n_local experts."""
    w13, w13_sf, w13_gs = random_nvfp4_experts(n_local, 2 * I, H, seed * 7919 + 1, device)
    w2, w2_sf, w2_gs = random_nvfp4_experts(n_local, H, I, seed * 7919 + 2, device)
    weights = {
        "w13": w13, "w13_sf": w13_sf.view(torch.float8_e4m3fn), "w13_gs": w13_gs,
        "w2": w2, "w2_sf": w2_sf.view(torch.float8_e4m3fn), "w2_gs": w2_gs,
    }
    if post_norm:
        gen = torch.Generator(device=device).manual_seed(seed * 7919 + 3)
        weights["post_norm_w"] = (torch.randn((H,), generator=gen, device=device) * 0.1).to(torch.bfloat16)
    return weights


def make_weights_random_bytes(H, I, n_local, seed, device):
    """Valid NVFP4 experts from random codes and scale bytes in the range the quantiser produces
    for N(0, 0.02) weights (0x63..0x7E). Cheap to build; used where only the cost of the math
    matters (timing the CPU oracle), not for parity."""
    gen = torch.Generator(device=device).manual_seed(seed * 7919 + 4)

    def mk(rows, K):
        codes = torch.randint(0, 256, (n_local, rows, K // 2), generator=gen, device=device, dtype=torch.uint8)
        sf = torch.randint(0x63, 0x7F, (n_local, rows, K // 16), generator=gen, device=device, dtype=torch.uint8)
        return codes, sf.view(torch.float8_e4m3fn)

    w13, w13_sf = mk(2 * I, H)
    w2, w2_sf = mk(H, I)
    gs = torch.full((n_local,), 2.0e-5, dtype=torch.float32, device=device)
    return {"w13": w13, "w13_sf": w13_sf, "w13_gs": gs, "w2": w2, "w2_sf": w2_sf, "w2_gs": gs.clone()}


def make_logits(T, E, kind, seed, device):
    """FP32 router logits [T, E]. uniform: U(0,1); normal: N(0,1); zipf: N(0,1) + log p_e with
    p_e ~ rank^-1.2 over a seeded permutation of the experts."""
    gen = torch.Generator(device=device).manual_seed(seed * 104729 + 5)
    if kind == "uniform":
        return torch.rand((T, E), generator=gen, device=device)
    noise = torch.randn((T, E), generator=gen, device=device)
    if kind == "normal":
        return noise
    if kind == "zipf":
        rank = torch.randperm(E, generator=gen, device=device).float() + 1.0
        logp = -1.2 * rank.log()
        logp = logp - torch.logsumexp(logp, 0)
        # at T = 8192, E = 128, top-8 this leaves a handful of experts empty and gives the
        # five most popular ones between 4800 and 8100 tokens each
        return noise + logp
    raise ValueError(kind)


def make_inputs(shape, T, seed, device, local_start=0, local_count=None):
    """Returns (data, extras): data is the reference's `Inputs` dict without ids/weights
    filled in unless routing is done here; extras holds logits or the router weight."""
    s = SHAPES[shape]
    H, E, k = s["H"], s["E"], s["k"]
    gen = torch.Generator(device=device).manual_seed(seed * 15485863 + 11)
    x = torch.randn((T, H), generator=gen, device=device).to(torch.bfloat16)
    cfg = {"bs": T, "d_hidden": H, "d_expert": s["I"], "n_experts": E, "local_start": local_start,
           "local_count": E if local_count is None else local_count, "top_k": k,
           "sharding": "none" if local_count in (None, E) else f"ep{E // local_count}"}
    data = {"hidden_states": x, "config": cfg}
    extras = {}
    if s["router"] == "weight":
        extras["router"] = torch.randn((E, H), generator=gen, device=device) * 0.02
    else:
        data["router_logits"] = make_logits(T, E, s["router"], seed, device)
    return data, extras


def algorithmic_bytes(H, I, E, k, T, touched_experts, router_in_module=False):
    """Bytes the step must move: touched experts' NVFP4 weights + x in + out + ids/weights."""
    w_e = 3 * I * H * (0.5 + 1.0 / 16.0) + 8
    b = touched_experts * w_e + 2 * T * H + 2 * T * H + 8 * T * k
    if router_in_module:
        b += 4 * E * H
    return b


def algorithmic_flops(H, I, routed_pairs):
    return 2.0 * routed_pairs * 3 * I * H
