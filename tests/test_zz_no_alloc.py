"""msk_moe_forward_static: the expert step for callers that must not allocate.

A host that has given all device memory to its own pool, or that calls this library while its
allocator is locked or from a thread that must not enter the driver's allocator, cannot provide the workspace
msk_moe_forward asks for. The static variant keeps that scratch in a device array inside the
library. This test calls it through the C ABI and compares it with msk_moe_forward and with the
CPU oracle on the same inputs, twice in a row (the second call finds the array as the first one
left it), and reads the array's own status word back through msk_moe_static_status.

Collected last on purpose (file name), so a failure here cannot hide any other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = 1e-2  # max|a - b| / max|b|, the bar of the other expert-output tests


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def test_forward_static_matches_forward_twice(cuda_dev):
    import muse_moe_w4a16 as moe
    from muse_moe_w4a16 import _lib, inputs
    from oracle import moe_oracle as orc

    lib = _lib.load()
    H, I, E, k = 1024, 512, 16, 4
    w = inputs.make_weights(H, I, E, 5, cuda_dev, post_norm=True)
    st = moe.prepare(w, n_experts=E, top_k=k, max_tokens=32)
    cfg = st["cfg"]
    for call, T in enumerate((7, 32)):
        g = torch.Generator(device=cuda_dev).manual_seed(100 + call)
        x = torch.randn((T, H), generator=g, device=cuda_dev).to(torch.bfloat16)
        logits = torch.randn((T, E), generator=g, device=cuda_dev)
        want, ids, tw = moe.kernel_fn({"hidden_states": x, "router_logits": logits}, st, return_routing=True)
        got = torch.full((T, H), float("nan"), dtype=torch.bfloat16, device=cuda_dev)
        rc = lib.msk_moe_forward_static(ctypes.byref(cfg), _lib.ptr(st["packed13"]), _lib.ptr(st["packed2"]),
                                        _lib.ptr(st["gs13"]), _lib.ptr(st["gs2"]), _lib.ptr(st["post_norm_w"]),
                                        _lib.ptr(x), _lib.ptr(ids), _lib.ptr(tw), _lib.ptr(got), T, _stream())
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all()
        err = float((got.float() - want.float()).abs().max() / want.float().abs().max())
        assert err <= TOL, (call, err)
        ref = orc.moe_forward(x, ids, tw, w).float()
        err_o = float((got.float().cpu() - ref).abs().max() / ref.abs().max())
        assert err_o <= TOL, (call, err_o)
        status = ctypes.c_int(-1)
        assert lib.msk_moe_static_status(ctypes.byref(status), _stream()) == 0
        assert status.value == 0          # no bounded wait of the static call gave up
    assert moe.read_status(st) == 0


def test_forward_static_rejects_sizes_beyond_its_array(cuda_dev):
    import muse_moe_w4a16 as moe
    from muse_moe_w4a16 import _lib, inputs

    lib = _lib.load()
    H, I, E, k = 512, 256, 8, 2
    w = inputs.make_weights(H, I, E, 6, cuda_dev)
    st = moe.prepare(w, n_experts=E, top_k=k, max_tokens=128)
    cfg = st["cfg"]
    T = 65  # 65 * 2 routed rows > 128
    x = torch.zeros((T, H), dtype=torch.bfloat16, device=cuda_dev)
    ids = torch.zeros((T, k), dtype=torch.int32, device=cuda_dev)
    tw = torch.zeros((T, k), dtype=torch.float32, device=cuda_dev)
    out = torch.zeros((T, H), dtype=torch.bfloat16, device=cuda_dev)
    rc = lib.msk_moe_forward_static(ctypes.byref(cfg), _lib.ptr(st["packed13"]), _lib.ptr(st["packed2"]),
                                    _lib.ptr(st["gs13"]), _lib.ptr(st["gs2"]), None, _lib.ptr(x), _lib.ptr(ids),
                                    _lib.ptr(tw), _lib.ptr(out), T, _stream())
    assert rc == -6  # MSK_ERR_TOO_LARGE
