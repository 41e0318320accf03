"""ctypes binding of libb200nodes.so.  The library is required: there is no fallback path."""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libb200nodes.so")

vp, i32, f32, sz = C.c_void_p, C.c_int, C.c_float, C.c_size_t


class MoeLists(C.Structure):
    _fields_ = [(n, vp) for n in ("counts", "offsets", "row_of_pair", "slot_of_row", "wt_of_row", "blk_expert",
                                  "blk_row0", "blk_rows", "nblocks")]


class MoeWeights(C.Structure):
    _fields_ = [(n, vp) for n in ("w13", "s13", "w2", "s2", "sh13", "shs13", "sh2", "shs2")]


# name -> (restype, argtypes); mirrors include/b200nodes.h
PROTOTYPES = {
    "b200_abi_version": (i32, []),
    "b200_last_error": (C.c_char_p, []),
    "b200_router_scratch_bytes": (sz, [i32, i32, i32]),
    "b200_router": (i32, [vp, vp, vp, i32, i32, i32, i32, i32, vp, vp, vp, vp, sz, vp]),
    "b200_router_static_max_scratch_bytes": (sz, []),
    "b200_router_static": (i32, [vp, vp, vp, i32, i32, i32, i32, i32, vp, vp, vp, vp]),
    "b200_moe_max_blocks": (i32, [i32, i32, i32, i32]),
    "b200_moe_build_lists": (i32, [vp, vp, vp, i32, i32, i32, i32, i32, i32, C.POINTER(MoeLists), vp]),
    "b200_moe_build_lists_range": (i32, [vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, C.POINTER(MoeLists), vp]),
    "b200_moe_w8a8_workspace_bytes": (sz, [i32, i32, i32, i32]),
    "b200_moe_w8a8": (i32, [vp, i32, i32, i32, i32, i32, C.POINTER(MoeWeights), C.POINTER(MoeLists), vp, vp, sz, vp,
                            vp, i32, vp, vp]),
    "b200_moe_w8a8_ep": (i32, [vp, i32, i32, i32, i32, i32, C.POINTER(MoeWeights), C.POINTER(MoeLists), C.POINTER(vp), i32,
                               i32, i32, vp, sz, vp, vp]),
    "b200_ep_push": (i32, [vp, vp, vp, i32, i32, i32, i32, i32, C.POINTER(vp), C.POINTER(vp), C.POINTER(vp), vp]),
    "b200_moe_fp8_workspace_bytes": (sz, [i32, i32, i32, i32]),
    "b200_moe_fp8": (i32, [vp, i32, i32, i32, i32, i32, C.POINTER(MoeWeights), C.POINTER(MoeLists), vp, vp, sz, vp,
                           i32, vp, vp]),
    "b200_moe_fp8_ep": (i32, [vp, i32, i32, i32, i32, i32, C.POINTER(MoeWeights), C.POINTER(MoeLists), C.POINTER(vp), i32,
                              i32, i32, vp, sz, vp, vp]),
    "b200_ep_barrier": (i32, [C.POINTER(vp), vp, i32, i32, i32, C.c_ulonglong, vp, vp]),
    "b200_ep_put": (i32, [vp, sz, sz, C.POINTER(vp), i32, vp]),
    "b200_set_wait_budget_ns": (i32, [C.c_ulonglong]),
    "b200_selftest_wait_expiry": (i32, [vp, vp]),
    "b200_dense_fp8_split": (i32, [vp, i32, i32, vp, vp, i32, i32, C.POINTER(i32), C.POINTER(vp), C.POINTER(i32), vp, sz,
                                   vp, vp]),
    "b200_dense_fp8_add_rmsnorm_workspace_bytes": (sz, [i32, i32, i32]),
    "b200_dense_fp8_add_rmsnorm": (i32, [vp, i32, i32, vp, vp, i32, vp, vp, f32, vp, vp, vp, sz, vp, vp]),
    "b200_moe_combine": (i32, [vp, vp, vp, vp, i32, i32, i32, vp, vp]),
    "b200_moe_combine_norm": (i32, [vp, vp, vp, vp, i32, i32, i32, vp, vp, vp, f32, vp, vp]),
    "b200_moe_combine_norm_q": (i32, [vp, vp, vp, vp, i32, i32, i32, vp, vp, vp, f32, vp, vp, vp, vp]),
    "b200_dense_fp8_split_q": (i32, [vp, vp, i32, i32, vp, vp, i32, i32, C.POINTER(i32), C.POINTER(vp), C.POINTER(i32), vp,
                                     vp]),
    "b200_attn_front_q": (i32, [vp, vp, i32, vp, vp, vp, vp, vp, vp, i32, f32, i32, vp, vp, vp, vp, vp, vp]),
    "b200_attn_front_workspace_bytes": (sz, [i32]),
    "b200_attn_front": (i32, [vp, i32, vp, vp, vp, vp, vp, vp, i32, f32, i32, vp, vp, vp, vp, vp, sz, vp, vp]),
    "b200_attn_verify_splits": (i32, [i32]),
    "b200_attn_verify_workspace_bytes": (sz, [i32, i32]),
    "b200_attn_verify": (i32, [vp, vp, vp, vp, vp, vp, i32, vp, i32, vp, i32, f32, i32, vp, vp, sz, vp, vp]),
    "b200_dense_fp8_workspace_bytes": (sz, [i32, i32]),
    "b200_dense_fp8": (i32, [vp, i32, i32, vp, vp, i32, vp, vp, sz, vp, vp]),
    "b200_add_rmsnorm": (i32, [vp, vp, vp, f32, i32, i32, vp, vp]),
    "b200_lmhead_workspace_bytes": (sz, [i32, i32, i32]),
    "b200_lmhead_argmax": (i32, [vp, i32, i32, vp, vp, i32, i32, vp, vp, vp, vp, sz, vp, vp]),
    "b200_argmax_merge": (i32, [vp, vp, i32, i32, vp, vp]),
    "b200_gdn_verify": (i32, [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, f32, i32, vp, vp, sz, vp, vp]),
    "b200_gdn_workspace_bytes": (sz, [i32]),
    "b200_gdn_ring_fold": (i32, [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, vp]),
    "b200_gdn_verify_replay": (i32, [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp,
                                     vp, f32, i32, vp, vp, sz, vp, vp]),
}

_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m bundles_b200.build` (nvcc, sm_100a). "
                "There is no CPU or PyTorch fallback.")
        _lib = C.CDLL(LIB_PATH)
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(_lib, name)
            fn.restype = res
            fn.argtypes = args
    return _lib


class B200Error(RuntimeError):
    pass


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = lib().b200_last_error().decode(errors="replace")
        raise B200Error(f"{what} failed with code {rc}: {msg}")
