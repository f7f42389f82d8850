"""ctypes binding of libbonsai_khq_b200.so -- the thin host shim over the C ABI.

The library is looked up the way the reference host does (``src/ops.mojo:585-611``):
``$BONSAI_CUDA_LIB`` first, then the in-tree build.  There is no CPU fallback: if the library
cannot be loaded every call raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_float, c_int, c_longlong, c_size_t, c_uint, c_void_p
from pathlib import Path

_PKG_DIR = Path(__file__).resolve().parent
LIB_NAME = "libbonsai_khq_b200.so"

# symbol -> (restype, argtypes).  Order and meaning follow include/khq_b200.h.
_P = c_void_p
SIGNATURES = {
    "bonsai_cuda_sm75_init": (c_int, []),
    "khq_state_slot": (c_void_p, [c_int]),
    "launch_khq_compress_fp16": (c_int, [_P] * 10 + [c_int, c_int, c_float, c_float, c_int, _P]),
    "launch_khq_attn_fp16": (
        c_int,
        [_P] * 18 + [c_int] * 5 + [c_int, c_float, c_float, c_float, c_float, c_int, c_int, _P],
    ),
    "launch_khq_attn_strided_fp16": (
        c_int,
        [_P] * 18 + [c_int] * 4 + [c_int, c_float, c_float, c_float, c_float, c_int, c_int, c_int, c_int, _P],
    ),
    "launch_khq_window_attn_fp16": (c_int, [_P] * 4 + [c_int] * 6 + [c_float, _P]),
    "launch_khq_merge_gate_fp16": (c_int, [_P] * 4 + [c_int, c_int, c_int, _P]),
    "launch_khq_gather_q_fp16": (c_int, [_P, _P, c_int, c_int, _P]),
    "khq_b200_plan_decode": (c_int, [_P, _P, c_int, c_int, _P, c_int, _P, _P]),
    "khq_b200_decode_workspace_bytes": (c_size_t, [c_int]),
    "launch_khq_decode_batched_fp16": (
        c_int, [_P, _P, _P, c_int, c_int, _P, c_size_t, c_int, c_float, c_float, c_int, c_int, _P]),
    "launch_khq_decode_batched_partial_fp16": (
        c_int, [_P, _P, _P, c_int, c_int, _P, c_size_t, c_int, c_float, c_float, c_int, c_int, _P, _P]),
    "launch_khq_attn_static_fp16": (
        c_int, [_P] * 17 + [c_int] * 5 + [c_float, c_float, c_float, c_float, c_int, c_int, _P]),
    "launch_khq_merge_slots_gate_fp16": (c_int, [_P, c_int, _P, _P, c_int, c_int, _P]),
    "launch_khq_decode_step_fp16": (c_int, [_P] * 25 + [c_int] * 5 + [c_float] * 4 + [_P]),
    "launch_khq_gqa_prefill_fp16": (
        c_int, [_P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_float, c_longlong, c_longlong, c_longlong, _P]),
    "launch_khq_gqa_prefill_tc5_fp16": (
        c_int, [_P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_float, c_longlong, c_longlong, c_longlong, _P]),
    "launch_khq_gqa_prefill_bf16": (
        c_int, [_P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_float, c_longlong, c_longlong, c_longlong, _P]),
    "launch_khq_gqa_prefill_mma_fp16": (
        c_int, [_P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_float, c_longlong, c_longlong, c_longlong, _P]),
    "khq_b200_prefill_select": (c_int, [c_int]),
    "khq_b200_prefill_tc5_items_per_cta": (c_int, [c_int]),
    "khq_b200_prefill_status": (c_int, []),
    "launch_khq_prestep_fp16": (c_int, [_P] * 8 + [c_int] * 5 + [c_float, c_float, c_int, _P]),
    "launch_khq_prestep_batched_fp16": (
        c_int, [_P] * 8 + [c_longlong, _P, _P] + [c_int] * 5 + [c_float, c_float, c_int, _P]),
    "launch_khq_compress_batched_fp16": (
        c_int, [_P, c_int, c_int] + [_P] * 9 + [c_int, c_float, c_float, c_int, c_longlong, _P]),
    "launch_khq_update_descs": (c_int, [_P, _P, c_int, c_int, _P]),
    "launch_khq_cal_kstatic_fp32": (c_int, [_P, c_int, _P, _P, _P, _P]),
    "khq_b200_version": (c_char_p, []),
    "khq_b200_device_status": (c_int, []),
    "khq_b200_device_status_clear": (c_int, []),
    "khq_b200_enable_peer_access": (c_int, [c_int]),
    "khq_b200_peer_alloc": (c_int, [c_size_t, POINTER(c_void_p), c_char_p]),
    "khq_b200_peer_open": (c_int, [c_char_p, POINTER(c_void_p)]),
    "khq_b200_peer_close": (c_int, [_P]),
    "khq_b200_peer_free": (c_int, [_P]),
    "khq_b200_peer_poke": (c_int, [_P, c_uint]),
    "khq_b200_peer_peek": (c_int, [_P, POINTER(c_uint)]),
    "launch_khq_publish_partials_fp32": (c_int, [_P, c_int, _P, _P, c_int, c_int, c_int, c_longlong, c_uint, _P]),
    "launch_khq_publish_bytes": (c_int, [_P, c_size_t, _P, c_longlong, _P, c_int, c_int, c_uint, _P]),
    "launch_khq_wait_flag": (c_int, [_P, c_uint, c_uint, _P]),
    "launch_khq_merge_slots_wait_gate_fp16": (c_int, [_P, _P, c_int, c_uint, c_int, _P, _P, c_int, c_int, c_uint, _P]),
}

_lib = None


class KhqLibraryError(RuntimeError):
    pass


def library_path() -> Path:
    env = os.environ.get("BONSAI_CUDA_LIB")
    return Path(env) if env else _PKG_DIR / LIB_NAME


def load() -> ctypes.CDLL:
    """Load the CUDA library once; raise loudly if it is missing (no fallback exists)."""
    global _lib
    if _lib is not None:
        return _lib
    path = library_path()
    if not path.exists():
        raise KhqLibraryError(
            f"{path} not found: build it with `python -m bonsai_mojo_1bit_optimization_t4_cuda_b200.build` "
            "(this package has no CPU or PyTorch fallback)"
        )
    lib = ctypes.CDLL(str(path), mode=ctypes.RTLD_GLOBAL)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means the build is stale
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def ptr(t) -> int:
    """Device address of a torch tensor (or pass an int / None through)."""
    if t is None:
        return 0
    if isinstance(t, int):
        return t
    return t.data_ptr()


def current_stream() -> int:
    import torch

    return torch.cuda.current_stream().cuda_stream


class KhqLaunchError(RuntimeError):
    def __init__(self, name: str, code: int):
        super().__init__(f"{name} returned {code}")
        self.code = code


def check(name: str, code: int) -> None:
    """The reference host raises instead of falling back when a launch fails
    (``src/models/qwen3_5/attention.mojo:359-365``); so does this one."""
    if code != 0:
        raise KhqLaunchError(name, code)
