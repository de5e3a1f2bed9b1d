"""ctypes binding of libmsk_moe.so (C ABI declared in include/msk_moe.h).

There is no fallback: if the library cannot be loaded or a call returns a non-zero
status, a RuntimeError is raised.
"""
import ctypes
import os
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("MSK_MOE_LIB", os.path.join(_HERE, "libmsk_moe.so"))  # override: a differently built library

ROUTE_SOFTMAX_TOPK = 0
ROUTE_SIGMOID_BIAS = 1

_ERRORS = {
    -1: "MSK_ERR_NULL: a required pointer is NULL",
    -2: "MSK_ERR_SHAPE: unsupported shape",
    -3: "MSK_ERR_ALIGN: pointer not 16-byte aligned",
    -4: "MSK_ERR_WORKSPACE: workspace too small",
    -5: "MSK_ERR_RANGE: local expert range outside [0, n_experts)",
    -6: "MSK_ERR_TOO_LARGE: size beyond a stated maximum",
}


class MskMoeCfg(ctypes.Structure):
    """Mirror of `struct MskMoeCfg` (include/msk_moe.h); field order and types must match."""

    _fields_ = [
        ("hidden", ctypes.c_int32),
        ("inter", ctypes.c_int32),
        ("n_experts", ctypes.c_int32),
        ("local_start", ctypes.c_int32),
        ("local_count", ctypes.c_int32),
        ("top_k", ctypes.c_int32),
        ("routing_mode", ctypes.c_int32),
        ("route_scale", ctypes.c_float),
        ("post_norm_eps", ctypes.c_float),
        ("num_ctas", ctypes.c_int32),
        ("decode_path", ctypes.c_int32),
        ("no_pdl", ctypes.c_int32),
        ("token_tile", ctypes.c_int32),
        ("max_tokens", ctypes.c_int32),
        ("trace", ctypes.c_int32),
        ("stop_after", ctypes.c_int32),
        ("flat_shares", ctypes.c_int32),
    ]

    def __deepcopy__(self, memo):
        c = MskMoeCfg()
        ctypes.memmove(ctypes.byref(c), ctypes.byref(self), ctypes.sizeof(MskMoeCfg))
        return c


_P = ctypes.c_void_p
_CFG = ctypes.POINTER(MskMoeCfg)
_SZP = ctypes.POINTER(ctypes.c_size_t)
_INTP = ctypes.POINTER(ctypes.c_int)

# name -> argtypes; every entry point returns int. Kept in one table so that the CPU test
# can check that the library exports exactly what the header declares.
SIGNATURES = {
    "msk_moe_packed_bytes": [_CFG, _SZP, _SZP],
    "msk_moe_repack": [_CFG, _P, _P, _P, _P, _P, _P, _P],
    "msk_moe_unpack": [_CFG, _P, _P, _P, _P, _P, _P, _P],
    "msk_moe_dequant_packed": [_CFG, _P, _P, _P, _P, _P],
    "msk_moe_router_logits": [_CFG, _P, _P, _P, ctypes.c_int, _P],
    "msk_moe_router_logits_hilo": [_CFG, _P, _P, _P, _P, ctypes.c_int, _P],
    "msk_moe_route": [_CFG, _P, _P, _P, _P, ctypes.c_int, _P],
    "msk_moe_sort": [_CFG, _P, ctypes.c_int, _P, _P, _P, _P, _P],
    "msk_moe_workspace_bytes": [_CFG, _SZP],
    "msk_moe_workspace_init": [_CFG, _P, ctypes.c_size_t, _P],
    "msk_moe_forward": [_CFG, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, ctypes.c_size_t, ctypes.c_int, _P],
    "msk_moe_forward_prenorm": [_CFG, _P, _P, _P, _P, _P, _P, ctypes.c_float, _P, _P, _P, _P, _P, _P, _P, ctypes.c_size_t,
                                ctypes.c_int, _P],
    "msk_moe_forward_logits": [_CFG, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, ctypes.c_size_t, ctypes.c_int, _P],
    "msk_moe_forward_timed": [_CFG, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, ctypes.c_size_t, ctypes.c_int, _P,
                              ctypes.POINTER(ctypes.c_float)],
    "msk_moe_forward_static": [_CFG, _P, _P, _P, _P, _P, _P, _P, _P, _P, ctypes.c_int, _P],
    "msk_moe_static_status": [_INTP, _P],
    "msk_moe_plan": [_CFG, ctypes.c_int, _INTP],
    "msk_moe_share_pieces": [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                             _INTP, ctypes.c_int, _INTP],
    "msk_moe_workspace_view": [_CFG, _P, ctypes.c_int, ctypes.POINTER(_P)],
    "msk_moe_read_status": [_P, _INTP, _P],
    "msk_moe_attrs": [ctypes.c_int, ctypes.c_int, _INTP],
    "msk_ep_combine": [_P, _P, ctypes.c_int, _P, ctypes.c_int, ctypes.c_int, _P, ctypes.c_int, ctypes.c_int, ctypes.c_int, _P],
    "msk_ep_flag_write": [_P, ctypes.c_uint32, _P],
    "msk_ep_flag_wait": [_P, ctypes.c_uint32, _P],
    "msk_l2_sweep": [_P, ctypes.c_size_t, _P, _P],
    "msk_bw_probe": [_P, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ctypes.c_int, _P, ctypes.c_int, _P],
}

_lock = threading.Lock()
_lib = None


def _build_module():
    import importlib.util

    spec = importlib.util.spec_from_file_location("_msk_build", os.path.join(os.path.dirname(_HERE), "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def load():
    """Load libmsk_moe.so once per process. The library carries a hash of the sources it was built
    from (msk_build_id); when it differs from the sources beside it (or the library is absent) the
    library is rebuilt with nvcc first, and if that is impossible the load fails: tests and
    benchmarks never run a binary that is older than the source tree."""
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        default_path = "MSK_MOE_LIB" not in os.environ
        if default_path:
            bm = _build_module()
            if bm.built_id(LIB_PATH) != bm.source_id():
                bm.build_library()      # raises when nvcc is missing or fails
        try:
            lib = ctypes.CDLL(LIB_PATH)
        except OSError as exc:  # no CPU fallback by design
            raise RuntimeError(f"muse_moe_w4a16: cannot load {LIB_PATH}: {exc}") from exc
        for name, argtypes in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = ctypes.c_int
        lib.msk_build_id.restype = ctypes.c_char_p
        lib.msk_build_id.argtypes = []
        _lib = lib
        return lib


def build_id():
    """Hash of the sources the loaded library was built from."""
    return load().msk_build_id().decode()


def check(status, what):
    """Raise RuntimeError on a non-zero C-ABI status."""
    if status == 0:
        return
    if status < 0:
        raise RuntimeError(f"{what}: {_ERRORS.get(status, 'error %d' % status)}")
    raise RuntimeError(f"{what}: CUDA error {status}")


class LibHandle:
    """Deep-copy-safe handle kept in `state` (the reference wraps its extension objects the same
    way because its harness deep-copies the state: muse_decode_layer/py/10_context_router.py:88-96)."""

    def __deepcopy__(self, memo):
        return self

    def __copy__(self):
        return self

    @property
    def lib(self):
        return load()


def ptr(t):
    """Device pointer of a tensor (or None)."""
    return None if t is None else ctypes.c_void_p(t.data_ptr())
