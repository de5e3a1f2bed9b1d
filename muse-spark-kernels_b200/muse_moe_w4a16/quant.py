"""NVFP4 quantiser used to build synthetic weights (torch ops; CPU or CUDA).

Format (the reference's input types, muse_moe_w4a16/py/00_moe_w4a16.py:72-80 and
py/01_build_pack.py:78-85): E2M1 codes two per byte with the low nibble holding the even k,
one E4M3 scale byte per 16 consecutive k, one FP32 global scale per matrix:
    W[r, k] = e2m1(code[r, k]) * e4m3(sf[r, k // 16]) * gs
Quantisation recipe of the benchmark configs: gs = amax / (6 * 448);
sf = e4m3_rn(block_amax / (6 * gs)); code = nearest E2M1 value of w / (sf * gs), ties to the
even code. This module only produces inputs; the library itself never requantises.
"""
import torch

E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
# decision boundaries between neighbouring magnitudes; a tie goes to the code with mantissa
# bit 0 (0, 1, 2, 4), which is what "<" vs "<=" encodes below
_BOUNDS = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)
_TIE_GOES_UP = (False, True, False, True, False, True, False)


def e2m1_codes(v):
    """Nearest E2M1 code (4 bits, sign in bit 3) of each element of fp32 tensor v."""
    a = v.abs()
    mag = torch.zeros_like(a, dtype=torch.uint8)
    for b, up in zip(_BOUNDS, _TIE_GOES_UP):
        mag += ((a >= b) if up else (a > b)).to(torch.uint8)
    sign = (v < 0).to(torch.uint8) << 3
    return mag | sign


def quantize_nvfp4(w):
    """w: [R, K] float tensor (K % 16 == 0) -> (codes uint8 [R, K/2], sf uint8 [R, K/16], gs fp32 scalar)."""
    w = w.float()
    R, K = w.shape
    amax = w.abs().max()
    gs = (amax / (6.0 * 448.0)).clamp_min(1e-30).float()
    blocks = w.view(R, K // 16, 16)
    bamax = blocks.abs().amax(-1)
    sf8 = (bamax / (6.0 * gs)).to(torch.float8_e4m3fn)
    sf = sf8.float()
    denom = (sf * gs).unsqueeze(-1)
    scaled = torch.where(denom > 0, blocks / denom, torch.zeros_like(blocks))
    codes = e2m1_codes(scaled).view(R, K)
    packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).contiguous()
    return packed, sf8.view(torch.uint8).contiguous(), gs


def random_nvfp4_experts(n_experts, rows, K, seed, device, std=0.02, chunk=8):
    """Per expert: BF16 ~ N(0, std) [rows, K] quantised to NVFP4. Returns (codes [E, rows, K/2],
    sf [E, rows, K/16] uint8, gs [E] fp32). Generated expert by expert to bound memory."""
    gen = torch.Generator(device=device).manual_seed(seed)
    codes = torch.empty((n_experts, rows, K // 2), dtype=torch.uint8, device=device)
    sf = torch.empty((n_experts, rows, K // 16), dtype=torch.uint8, device=device)
    gs = torch.empty((n_experts,), dtype=torch.float32, device=device)
    for e in range(n_experts):
        w = (torch.randn((rows, K), generator=gen, device=device) * std).to(torch.bfloat16)
        c, s, g = quantize_nvfp4(w)
        codes[e], sf[e], gs[e] = c, s, g
    return codes, sf, gs
