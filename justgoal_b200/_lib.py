"""ctypes binding of libb200moe.so (the C ABI in include/b200moe.h).

There is no fallback: if the shared library is missing or does not load, importing this
module raises.  Build it with `python -m justgoal_b200.build`.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# B200MOE_LIB selects another build of the library (A/B timing of kernel variants); default: the in-tree build
LIB_PATH = os.environ.get("B200MOE_LIB") or os.path.join(HERE, "libb200moe.so")


class Config(C.Structure):
    _fields_ = [("hidden", C.c_int), ("intermediate", C.c_int), ("num_experts", C.c_int),
                ("num_local_experts", C.c_int), ("top_k", C.c_int), ("n_group", C.c_int),
                ("topk_group", C.c_int), ("routing_mode", C.c_int)]


class WsLayout(C.Structure):
    _fields_ = [(n, C.c_size_t) for n in (
        "status", "counts", "expert_row0", "tile_prefix", "topk_idx", "topk_w", "pair_row", "row_token",
        "row_w", "a_perm", "a_scale_perm", "act_hi", "act_lo", "act_scale", "y", "sk_count", "slices", "sk_partial", "trace",
        "tok_count", "rows_cap", "token_tile",
        "total_bytes")]


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} not found: build it with `python -m justgoal_b200.build` "
                          "(there is no CPU or PyTorch fallback for this operator)")
    lib = C.CDLL(LIB_PATH)
    vp, i, f, sz = C.c_void_p, C.c_int, C.c_float, C.c_size_t
    lib.b200moe_create.argtypes = [C.POINTER(Config), C.POINTER(vp)]
    lib.b200moe_destroy.argtypes = [vp]
    lib.b200moe_workspace_bytes.argtypes = [vp, i, C.POINTER(sz)]
    lib.b200moe_workspace_layout.argtypes = [vp, i, C.POINTER(WsLayout)]
    lib.b200moe_forward.argtypes = [vp] + [vp] * 8 + [i, i, f, vp, vp, sz, vp]
    lib.b200moe_route.argtypes = [vp, vp, vp, i, f, vp, vp, vp]
    lib.b200moe_forward_routed.argtypes = [vp, vp, vp] + [vp] * 6 + [i, i, vp, i, vp, sz, vp]
    lib.b200moe_ep_combine.argtypes = [vp, vp, vp, i, i, vp, vp]
    lib.b200moe_ep_row_bytes.argtypes = [vp, C.POINTER(i)]
    pv = C.POINTER(C.c_void_p)
    lib.b200moe_ep_push.argtypes = [vp, vp, vp, vp, vp, i, i, i, i, pv, vp]
    lib.b200moe_ep_barrier.argtypes = [vp, pv, i, i, C.c_uint, vp, vp]
    lib.b200moe_ep_unpack_slots.argtypes = [vp, vp, i, vp, vp, vp, vp, vp]
    lib.b200moe_ep_return.argtypes = [vp, vp, vp, i, i, i, pv, vp]
    lib.b200moe_ep_combine_slots.argtypes = [vp, vp, vp, i, i, i, vp, vp]
    lib.b200moe_forward_routed_slots.argtypes = [vp, vp] + [vp] * 4 + [i, i, i, i, pv, vp, sz, vp]
    lib.b200moe_ep_pack.argtypes = [vp, vp, vp, vp, vp, vp, i, i, vp, vp]
    lib.b200moe_ep_unpack.argtypes = [vp, vp, i, vp, vp, vp, vp, vp]
    lib.b200moe_set_wait_limit_ns.argtypes = [vp, C.c_ulonglong]
    lib.b200moe_quantize_1x128.argtypes = [vp, i, i, vp, vp, vp]
    lib.b200moe_status.argtypes = [vp, vp, vp, C.POINTER(i)]
    lib.b200moe_set_fused_combine.argtypes = [vp, i]
    lib.b200moe_set_tma_gather.argtypes = [vp, i]
    lib.b200moe_set_token_tile.argtypes = [vp, i]
    lib.b200moe_launches_per_forward.argtypes = [vp, i, C.POINTER(i)]
    lib.b200moe_launches_routed.argtypes = [vp, i, C.POINTER(i)]
    lib.b200moe_permute_noalloc.argtypes = [vp, vp, vp, i, i, vp, vp, vp, i, vp]
    lib.b200moe_profile_enable.argtypes = [vp, i]
    lib.b200moe_profile_read.argtypes = [vp, i, C.POINTER(f)]
    lib.b200moe_strerror.argtypes = [i]
    lib.b200moe_strerror.restype = C.c_char_p
    lib.b200moe_num_sms.argtypes = []
    for name in ("create", "destroy", "workspace_bytes", "workspace_layout", "forward", "route",
                 "forward_routed", "status", "set_fused_combine", "set_tma_gather", "set_token_tile", "launches_per_forward", "launches_routed", "num_sms", "profile_enable",
                 "profile_read", "permute_noalloc", "ep_combine", "ep_row_bytes", "ep_pack", "ep_unpack", "ep_push", "ep_barrier", "ep_unpack_slots",
                 "ep_return", "ep_combine_slots", "forward_routed_slots", "quantize_1x128", "set_wait_limit_ns"):
        getattr(lib, "b200moe_" + name).restype = i
    return lib


NOALLOC_MAX_TOKENS = 8192   # B200MOE_NOALLOC_MAX_TOKENS in include/b200moe.h

lib = _load()


class B200MoEError(RuntimeError):
    pass


def check(rc: int, what: str = "b200moe"):
    if rc != 0:
        raise B200MoEError(f"{what} failed with code {rc}: {lib.b200moe_strerror(rc).decode()}")
