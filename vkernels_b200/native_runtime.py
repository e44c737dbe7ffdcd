"""Locating and loading ``libvkernels_b200.so`` (ctypes).

Mirrors the reference's ``native_runtime.find_library`` lookup order
(src/python/vkernels/native_runtime.py:10-26): an explicit ``VKERNELS_LIB``
path first, then the in-tree build. There is no CPU fallback: when the library
cannot be loaded every op raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_int32, c_size_t, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
IN_TREE = os.path.join(_HERE, "lib", "libvkernels_b200.so")

_lib = None


def find_library() -> str | None:
    env = os.environ.get("VKERNELS_LIB")
    if env:
        return env if os.path.exists(env) else None
    return IN_TREE if os.path.exists(IN_TREE) else None


_SIGNATURES = {
    # name: (restype, [argtypes])
    "vk_version": (ctypes.c_char_p, []),
    "vk_has_cuda": (c_int, []),
    "vk_last_error": (ctypes.c_char_p, []),
    "vk_last_error_code": (c_int, []),
    "vk_set_last_error": (None, [c_int, ctypes.c_char_p]),
    "vk_hip_fused_moe_mxfp4": (None, [c_void_p] * 9 + [c_int] * 4 + [c_void_p] * 2 + [c_int, c_float,
                                      c_int, c_float, c_float, c_void_p, c_void_p, c_int, c_void_p]),
    "vk_hip_moe_align_block_size": (c_int, [c_void_p, c_void_p] + [c_int32] * 6 + [c_void_p] * 4),
    "vk_cuda_moe_align_block_size_noalloc": (c_int, [c_void_p, c_void_p] + [c_int32] * 6 + [c_void_p] * 4),
    "vk_fused_moe_mxfp4": (c_int32, [c_void_p] * 10 + [c_int] * 6 + [c_float, c_int, c_float, c_float,
                                     c_void_p, c_void_p]),
    "vk_moe_align_block_size": (c_int32, [c_void_p] + [c_int32] * 4 + [c_void_p] * 3),
    "vk_moe_align_block_size_max_em": (c_size_t, [c_int32] * 4),
    "vk_cuda_fused_moe_mxfp4_sorted_w": (c_int, [c_void_p] * 8 + [c_int] * 4 + [c_void_p] * 2 +
                                         [c_int, c_float, c_int, c_float, c_float, c_void_p, c_void_p,
                                          c_int, c_void_p]),
    "vk_cuda_fused_moe_mxfp4_bf16": (c_int, [c_void_p] * 8 + [c_int] * 4 + [c_void_p] * 2 +
                                     [c_int, c_float, c_int, c_float, c_float, c_void_p, c_void_p, c_int, c_void_p]),
    "vk_cuda_moe_workspace_bytes_bf16": (c_size_t, [c_int] * 5),
    "vk_cuda_moe_prepack_sizes": (c_int, [c_int] * 4 + [c_void_p] * 2),
    "vk_cuda_moe_prepack_weights": (c_int, [c_int] + [c_void_p] * 2 + [c_int] * 3 + [c_void_p] * 4),
    "vk_cuda_fused_moe_mxfp4_bf16_prepacked": (c_int, [c_void_p] * 8 + [c_int] * 4 + [c_void_p] * 2 +
                                               [c_int, c_float, c_int, c_float, c_float, c_void_p, c_void_p, c_int,
                                                c_void_p]),
    "vk_cuda_moe_router_logits": (c_int, [c_void_p] * 3 + [c_int] * 3 + [c_void_p]),
    "vk_cuda_moe_route_topk": (c_int, [c_void_p] * 2 + [c_int] * 7 + [c_float, c_int] + [c_void_p] * 3),
    "vk_cuda_moe_route_align_small": (c_int, [c_void_p] * 2 + [c_int] * 7 + [c_float] + [c_int] * 3 + [c_void_p] * 6),
    "vk_cuda_moe_set_impl": (c_int, [c_int]),
    "vk_cuda_moe_get_impl": (c_int, []),
    "vk_cuda_moe_workspace_bytes": (c_size_t, [c_int] * 5),
    "vk_cuda_moe_reserve_workspace": (c_int, [c_size_t]),
    "vk_cuda_moe_reserve_workspace_on": (c_int, [c_size_t, c_void_p]),
    "vk_cuda_moe_release_workspaces": (c_int, []),
    "vk_cuda_moe_workspace_live_bytes": (c_size_t, []),
    "vk_cuda_moe_kernel_status": (c_int, []),
    "vk_cuda_moe_reset_kernel_status": (c_int, []),
    "vk_cuda_moe_test_wait_timeout": (c_int, [ctypes.c_longlong, c_void_p]),
    "vk_cuda_mxfp4_dequant_rows_path": (c_int, [c_void_p] * 3 + [c_int] * 3 + [c_void_p]),
    "vk_cuda_moe_timing_begin": (c_int, [c_int]),
    "vk_cuda_moe_timing_end": (c_int, [c_void_p] * 3),
    "vk_cuda_mxfp4_dequant_rows": (c_int, [c_void_p] * 3 + [c_int] * 2 + [c_void_p]),
    "vk_cuda_moe_ep_pack": (c_int, [c_void_p] * 3 + [c_int] * 6 + [c_void_p] * 6 + [c_int, c_void_p]),
    "vk_cuda_moe_ep_combine": (c_int, [c_void_p] * 2 + [c_int] * 3 + [c_void_p] * 3),
    "vk_cuda_moe_ep_pack_meta": (c_int, [c_void_p] * 2 + [c_int] * 5 + [c_void_p] * 4),
    "vk_cuda_moe_ep_unpack_meta": (c_int, [c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int] +
                                   [c_void_p] * 5),
    "vk_cuda_moe_gateup_preact": (c_int, [c_void_p] * 6 + [c_int] * 7 + [c_void_p]),
    "vk_cuda_moe_act_epilogue": (c_int, [c_void_p] * 5 + [c_int] * 4 + [c_float, c_int, c_float, c_float, c_void_p]),
    "vk_cuda_moe_down_preact": (c_int, [c_void_p] * 6 + [c_int] * 7 + [c_void_p]),
    "vk_cuda_moe_combine": (c_int, [c_void_p] * 6 + [c_int] * 4 + [c_void_p]),
    "vk_cuda_moe_ep_pack_meta_peer": (c_int, [c_void_p] * 2 + [c_int] * 5 + [c_void_p] * 4 + [c_int, c_void_p]),
    "vk_cuda_moe_ep_unpack_meta_peer": (c_int, [c_void_p] * 2 + [c_int] * 3 + [c_void_p] * 2 + [c_int] * 2 +
                                        [c_void_p] * 5),
    "vk_cuda_fused_moe_mxfp4_rows_store": (c_int, [c_void_p] * 8 + [c_int] * 4 + [c_void_p] * 2 +
                                           [c_int, c_float, c_int, c_float, c_float, c_void_p, c_void_p,
                                            c_int, c_void_p]),
    "vk_cuda_moe_ep_combine_slots": (c_int, [c_void_p] * 3 + [c_int] * 4 + [c_void_p] * 3),
    "vk_cuda_moe_ep_flag_barrier": (c_int, [c_void_p, c_int, c_int, c_int, c_int, ctypes.c_longlong, c_void_p, c_void_p]),
    "vk_cuda_fused_moe_mxfp4_rows": (c_int, [c_void_p] * 8 + [c_int] * 4 + [c_void_p] * 2 +
                                     [c_int, c_float, c_int, c_float, c_float, c_void_p, c_void_p,
                                      c_int, c_void_p]),
}

EXPORTED = tuple(_SIGNATURES)


def load_library() -> ctypes.CDLL:
    """Load (once) and type the library. Raises ``RuntimeError`` if it is absent."""
    global _lib
    if _lib is None:
        path = find_library()
        if path is None:
            raise RuntimeError(
                "libvkernels_b200.so not found: build it with `python -m vkernels_b200.build` "
                "or point VKERNELS_LIB at it. There is no CPU fallback.")
        lib = ctypes.CDLL(path)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(lib, name, None)
            if fn is None:
                raise RuntimeError(f"{path} does not export {name}; rebuild the library")
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def last_error() -> str:
    return (load_library().vk_last_error() or b"").decode("utf-8", "replace")


def check(rc: int, what: str) -> None:
    """Raise for a non-zero status: ValueError for argument errors, RuntimeError otherwise."""
    if rc == 0:
        return
    msg = f"{what}: {last_error()} (status {rc})"
    raise ValueError(msg) if rc in (1, 2) else RuntimeError(msg)
