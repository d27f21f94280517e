"""ctypes binding of libmoe_b200.so -- the C ABI declared in include/moe_b200.h.

The library is loaded lazily and exactly once. There is no fallback: if the shared object is
missing or a call returns an error code, a RuntimeError is raised.
"""
import ctypes
import os
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
# MOE_B200_LIB points at a library built elsewhere (e.g. a variant under test); default: in-tree
LIB_PATH = os.environ.get("MOE_B200_LIB") or os.path.join(_HERE, "libmoe_b200.so")

_c_i32, _c_i64, _c_vp, _c_sz = ctypes.c_int32, ctypes.c_int64, ctypes.c_void_p, ctypes.c_size_t

# name -> (restype, argtypes); mirrors include/moe_b200.h one to one.
SIGNATURES = {
    "moe_b200_abi_version": (_c_i32, []),
    "moe_b200_error_string": (ctypes.c_char_p, [_c_i32]),
    "moe_b200_l_cap": (_c_i64, [_c_i64, _c_i32]),
    "moe_b200_dispatch_scratch_bytes": (_c_sz, [_c_i64, _c_i32]),
    "moe_b200_router_topk": (
        ctypes.c_int, [_c_vp, _c_i64, _c_i32, _c_i32, _c_i32, _c_i32, _c_vp, _c_vp, _c_vp, _c_vp]),
    "moe_b200_router_topk_bwd": (
        ctypes.c_int,
        [_c_vp, _c_vp, _c_vp, _c_vp, _c_i64, _c_i32, _c_i32, _c_i32, _c_i32, _c_vp, _c_vp]),
    "moe_b200_router_fused": (
        ctypes.c_int,
        [_c_vp, _c_i32, _c_vp, _c_vp, _c_i64, _c_i32, _c_i32, _c_i32, _c_i32, _c_i32, _c_vp, _c_vp, _c_vp,
         _c_vp]),
    "moe_b200_router_fused_bwd": (
        ctypes.c_int,
        [_c_vp, _c_i32, _c_vp, _c_vp, _c_vp, _c_vp, _c_i64, _c_i32, _c_i32, _c_i32, _c_i32, _c_i32, _c_vp,
         _c_vp, ctypes.c_float, _c_vp, _c_i32, _c_vp]),
    "moe_b200_balance_loss": (
        ctypes.c_int, [_c_vp, _c_vp, _c_i32, _c_i64, ctypes.c_float, _c_vp, _c_vp]),
    "moe_b200_dispatch": (
        ctypes.c_int,
        [_c_vp, _c_i64, _c_i32, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_sz, _c_i32,
         _c_i32, _c_vp, _c_vp]),
    "moe_b200_dispatch_static_max_pairs": (_c_i64, [_c_i32]),
    "moe_b200_router_dispatch_scratch_bytes": (_c_sz, [_c_i64, _c_i32]),
    "moe_b200_router_dispatch": (
        ctypes.c_int,
        [_c_vp, _c_i32, _c_vp, _c_vp, _c_i64, _c_i32, _c_i32, _c_i32, _c_i32, _c_i32, _c_vp, _c_vp, _c_vp,
         _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_sz, _c_vp, _c_vp]),
    "moe_b200_dispatch_static": (
        ctypes.c_int,
        [_c_vp, _c_i64, _c_i32, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp]),
    "moe_b200_permute": (
        ctypes.c_int, [_c_vp, _c_i64, _c_i32, _c_i32, _c_vp, _c_vp, _c_i64, _c_vp, _c_vp]),
    "moe_b200_combine": (
        ctypes.c_int, [_c_vp, _c_vp, _c_i64, _c_i32, _c_i32, _c_vp, _c_vp, _c_vp, _c_vp]),
    "moe_b200_segment_colsum": (
        ctypes.c_int,
        [_c_vp, _c_i64, _c_i32, _c_vp, _c_vp, _c_vp, _c_i32, _c_vp, _c_vp, _c_i64, _c_vp, _c_i64,
         _c_i32, _c_vp, _c_vp]),
    "moe_b200_group_sumsq": (ctypes.c_int, [_c_vp, _c_i32, _c_i64, _c_vp, _c_vp]),
    "moe_b200_axpby": (
        ctypes.c_int,
        [_c_vp, _c_vp, _c_vp, _c_i32, _c_i64, ctypes.c_float, ctypes.c_float, _c_vp,
         ctypes.c_float, _c_vp]),
    "moe_b200_rmsnorm": (
        ctypes.c_int, [_c_vp, _c_vp, _c_i64, _c_i32, ctypes.c_float, _c_vp, _c_vp, _c_vp]),
    "moe_b200_rmsnorm_bwd": (
        ctypes.c_int, [_c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_i64, _c_i32, _c_vp, _c_vp, _c_vp]),
    "moe_b200_copy_cols": (
        ctypes.c_int, [_c_vp, _c_i64, _c_i32, _c_i32, _c_vp, _c_i32, _c_vp]),
    "moe_b200_up_gemm": (
        ctypes.c_int,
        [_c_vp, _c_i64, _c_i32, _c_vp, _c_i32, _c_vp, _c_i32, _c_i32, _c_vp, _c_vp, _c_i32, _c_vp,
         _c_i32, _c_i64, _c_i32, _c_vp, _c_vp, _c_vp, _c_i64, _c_vp, _c_vp, _c_vp, _c_vp]),
    "moe_b200_down_gemm": (
        ctypes.c_int,
        [_c_vp, _c_i64, _c_i32, _c_vp, _c_i32, _c_vp, _c_i32, _c_i32, _c_vp, _c_vp, _c_i32, _c_vp,
         _c_vp, _c_i64, _c_vp, _c_vp, _c_vp, _c_vp]),
    "moe_b200_down_gemm_acc": (
        ctypes.c_int,
        [_c_vp, _c_i64, _c_i32, _c_vp, _c_i32, _c_vp, _c_i32, _c_i32, _c_vp, _c_vp, _c_i32, _c_vp,
         _c_vp, _c_i64, _c_i32, _c_vp, _c_i64, _c_vp, _c_vp, _c_vp]),
    "moe_b200_down_gemm_sum": (
        ctypes.c_int,
        [_c_vp, _c_i64, _c_i32, _c_vp, _c_i32, _c_i32, _c_vp, _c_i64, _c_vp, _c_vp, _c_vp]),
    "moe_b200_dx_gemm_sum": (
        ctypes.c_int,
        [_c_vp, _c_i64, _c_i32, _c_vp, _c_i32, _c_i32, _c_vp, _c_i64, _c_vp, _c_vp, _c_vp]),
    "moe_b200_dx_gemm_acc": (
        ctypes.c_int,
        [_c_vp, _c_i64, _c_i32, _c_vp, _c_i32, _c_vp, _c_i32, _c_i32, _c_vp, _c_vp, _c_i32, _c_vp,
         _c_i64, _c_i32, _c_vp, _c_i64, _c_vp, _c_vp, _c_vp]),
    "moe_b200_dhidden_glu_bwd": (
        ctypes.c_int,
        [_c_vp, _c_i64, _c_i32, _c_vp, _c_i32, _c_vp, _c_i32, _c_i32, _c_vp, _c_vp, _c_i32, _c_vp,
         _c_i32, _c_vp, _c_i64, _c_vp, _c_i32, _c_vp, _c_vp, _c_vp, _c_vp, _c_i64, _c_vp, _c_vp,
         _c_vp]),
    "moe_b200_dx_gemm": (
        ctypes.c_int,
        [_c_vp, _c_i64, _c_i32, _c_vp, _c_i32, _c_vp, _c_i32, _c_i32, _c_vp, _c_vp, _c_i32, _c_vp,
         _c_vp, _c_vp]),
    "moe_b200_wgrad_scratch_bytes": (
        ctypes.c_int,
        [_c_i32, _c_i32, _c_i64, _c_i32, _c_i32, _c_i32, ctypes.POINTER(_c_sz)]),
    "moe_b200_block_fwd_scratch_bytes": (_c_sz, [_c_i64, _c_i32, _c_i32, _c_i32, _c_i32, _c_i32]),
    "moe_b200_block_bwd_scratch_bytes": (_c_sz, [_c_i64, _c_i32, _c_i32, _c_i32, _c_i32, _c_i32]),
    "moe_b200_block_infer_scratch_bytes": (_c_sz, [_c_i64, _c_i32, _c_i32, _c_i32, _c_i32, _c_i32]),
    "moe_b200_block_infer": (
        ctypes.c_int,
        [_c_vp, _c_i64, _c_i32, _c_vp, _c_vp, _c_vp, _c_vp, _c_i32, _c_i32, _c_vp, _c_vp, _c_i32,
         _c_i32, _c_i32, _c_i32, _c_vp, _c_i32, _c_vp, _c_vp, _c_sz, ctypes.POINTER(_c_i32), _c_vp,
         _c_vp]),
    "moe_b200_block_fwd": (
        ctypes.c_int,
        [_c_vp, _c_i64, _c_i32, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_i32, _c_i32, _c_vp, _c_vp,
         _c_i32, _c_i32, _c_i32, _c_i32, ctypes.c_float, _c_i32,
         _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp,
         _c_vp, _c_vp, _c_vp, _c_sz, ctypes.POINTER(_c_i32), _c_vp, _c_vp]),
    "moe_b200_block_bwd": (
        ctypes.c_int,
        [_c_vp, _c_vp, _c_vp, _c_i64, _c_i32, _c_vp, _c_vp, _c_vp, _c_vp, _c_i32, _c_i32, _c_vp,
         _c_vp, _c_i32, _c_i32, _c_i32, _c_i32, ctypes.c_float, _c_i32,
         _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp,
         _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_sz, _c_vp, _c_vp,
         ctypes.POINTER(_c_i32), _c_vp, _c_vp]),
    "moe_b200_ep_plan": (
        ctypes.c_int, [_c_vp, _c_vp, _c_i32, _c_i32, _c_i32, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp,
                       _c_vp, _c_i64, _c_vp]),
    "moe_b200_ep_pair_map": (
        ctypes.c_int, [_c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_i64, _c_i32, _c_i32, _c_i32, _c_vp,
                       _c_vp, _c_vp]),
    "moe_b200_ep_push_rows": (
        ctypes.c_int, [_c_vp, _c_i64, _c_i32, _c_i32, _c_vp, _c_vp, _c_vp, _c_i64, _c_vp, _c_vp,
                       _c_vp, _c_vp, _c_vp, _c_i32, _c_vp, _c_vp]),
    "moe_b200_ep_pad_fix": (
        ctypes.c_int, [_c_vp, _c_vp, _c_i32, _c_vp, _c_i32, _c_vp, _c_i32, _c_vp]),
    "moe_b200_ep_pull_combine": (
        ctypes.c_int, [_c_vp, _c_i32, _c_vp, _c_vp, _c_i64, _c_i32, _c_i32, _c_vp, _c_vp, _c_vp]),
    "moe_b200_ep_pull_vec": (
        ctypes.c_int, [_c_vp, _c_i32, _c_vp, _c_vp, _c_i64, _c_i32, _c_i32, _c_vp, _c_vp]),
    "moe_b200_wgrad": (
        ctypes.c_int,
        [_c_vp, _c_i32, _c_i32, _c_vp, _c_i32, _c_i32, _c_i64, _c_vp, _c_i32, _c_i32, _c_vp, _c_i32,
         _c_i64, _c_i32, _c_vp, _c_i32, _c_vp, _c_vp, _c_sz, _c_vp, _c_i64, _c_i32, _c_vp, _c_vp]),
}

_lib = None
_lock = threading.Lock()


def load() -> ctypes.CDLL:
    """Load libmoe_b200.so (built by `python -m nanospeaker_b200.build`) and bind every symbol."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m nanospeaker_b200.build`. "
                "The MoE block has no non-CUDA implementation to fall back to."
            )
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError here = header and library disagree
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def error_string(code: int) -> str:
    return load().moe_b200_error_string(code).decode()


def check(code: int, what: str) -> None:
    """Turn a MOE_B200_ERR_* return code into a RuntimeError."""
    if code != 0:
        raise RuntimeError(f"{what} failed: {error_string(code)} (code {code})")


def ptr(t) -> int:
    """Device pointer of a tensor, or NULL for None."""
    return 0 if t is None else t.data_ptr()
