"""ctypes binding of ``libdtb200_attn.so`` (the C ABI declared in ``include/dtb200_attn.h``).

The library is the only compute path: if it is missing and cannot be built, or a call
returns a non-zero status, an exception is raised.  There is no CPU or PyTorch fallback.
"""
from __future__ import annotations

import ctypes
import os
import threading

from . import build as _build

DTB_OK = 0
STATUS_NAMES = {
    0: "DTB_OK", 1: "DTB_ERR_NULL", 2: "DTB_ERR_DTYPE", 3: "DTB_ERR_SHAPE", 4: "DTB_ERR_ALIGN",
    5: "DTB_ERR_ARCH", 6: "DTB_ERR_WORKSPACE", 7: "DTB_ERR_LAUNCH", 8: "DTB_ERR_TIMEOUT",
    9: "DTB_ERR_UNSUPPORTED",
}

FLAG_ZERO_PADDED_ROWS = 0x1
FLAG_BOUNDED_LOGITS = 0x2
FLAG_QK_FP8 = 0x8
STATIC_SCRATCH_BYTES = 32 << 20

# Every symbol the public header declares; tests check that the library exports all of them.
EXPORTED_SYMBOLS = (
    "dtb_version", "dtb_status_string", "dtb_last_error_detail", "dtb_attn_supported", "dtb_attn_workspace_bytes",
    "dtb_attn_fwd", "dtb_attn_launch_plan", "dtb_attn_fwd_static_scratch", "dtb_attn_fwd_scatter", "dtb_attn_fwd_sparse", "dtb_scatter_heads",
    "dtb_attn_fwd_residual", "dtb_attn_finalize", "dtb_fixed_m_operands", "dtb_qk_prepass", "dtb_quantize_e4m3",
    "dtb_smooth_k", "dtb_smooth_k_scratch_bytes", "dtb_fixed_m_from_norms", "dtb_out_proj", "dtb_sum_partials",
    "dtb_selftest_tmem_roundtrip", "dtb_selftest_qk", "dtb_selftest_pv", "dtb_selftest_wait_timeout",
)


class AttnParams(ctypes.Structure):
    """Mirror of ``dtb_attn_params``."""

    _fields_ = [
        ("q", ctypes.c_void_p), ("k", ctypes.c_void_p), ("v", ctypes.c_void_p), ("o", ctypes.c_void_p),
        ("B", ctypes.c_int32), ("Hq", ctypes.c_int32), ("Hkv", ctypes.c_int32),
        ("Sq", ctypes.c_int32), ("Skv", ctypes.c_int32), ("D", ctypes.c_int32),
        ("q_stride_b", ctypes.c_int64), ("q_stride_h", ctypes.c_int64), ("q_stride_s", ctypes.c_int64),
        ("k_stride_b", ctypes.c_int64), ("k_stride_h", ctypes.c_int64), ("k_stride_s", ctypes.c_int64),
        ("v_stride_b", ctypes.c_int64), ("v_stride_h", ctypes.c_int64), ("v_stride_s", ctypes.c_int64),
        ("o_stride_b", ctypes.c_int64), ("o_stride_h", ctypes.c_int64), ("o_stride_s", ctypes.c_int64),
        ("kv_len", ctypes.c_void_p), ("mk", ctypes.c_void_p),
        ("scale", ctypes.c_float), ("flags", ctypes.c_uint32), ("num_splits", ctypes.c_int32),
        ("status", ctypes.c_void_p),
    ]


class AttnResidual(ctypes.Structure):
    """Mirror of ``dtb_attn_residual``."""

    _fields_ = [
        ("o_acc", ctypes.c_void_p), ("m", ctypes.c_void_p), ("l", ctypes.c_void_p),
        ("kv_offset", ctypes.c_int32), ("q_offset", ctypes.c_int32), ("init", ctypes.c_int32),
    ]


class AttnScatter(ctypes.Structure):
    """Mirror of ``dtb_attn_scatter``."""

    _fields_ = [
        ("out_ptrs", ctypes.c_void_p * 8), ("n_peers", ctypes.c_int32), ("shard_rows", ctypes.c_int32),
        ("head_offset", ctypes.c_int32), ("total_heads", ctypes.c_int32),
        ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_size_t),
    ]


class ScatterHeadsParams(ctypes.Structure):
    """Mirror of ``dtb_scatter_heads_params``."""

    _fields_ = [
        ("src", ctypes.c_void_p * 3),
        ("stride_b", ctypes.c_int64 * 3), ("stride_h", ctypes.c_int64 * 3), ("stride_s", ctypes.c_int64 * 3),
        ("dst", (ctypes.c_void_p * 8) * 3),
        ("n_tensors", ctypes.c_int32), ("n_peers", ctypes.c_int32), ("rank", ctypes.c_int32),
        ("B", ctypes.c_int32), ("H", ctypes.c_int32), ("S_local", ctypes.c_int32), ("D", ctypes.c_int32),
    ]


class BlockTable(ctypes.Structure):
    """Mirror of ``dtb_block_table``."""

    _fields_ = [
        ("kv_table", ctypes.c_void_p), ("kv_count", ctypes.c_void_p), ("head_class", ctypes.c_void_p),
        ("n_classes", ctypes.c_int32), ("q_blocks", ctypes.c_int32), ("width", ctypes.c_int32),
    ]


class PrepassParams(ctypes.Structure):
    """Mirror of ``dtb_prepass_params``."""

    _fields_ = [
        ("q_in", ctypes.c_void_p), ("k_in", ctypes.c_void_p), ("v_in", ctypes.c_void_p),
        ("q_strides", ctypes.c_int64 * 3), ("k_strides", ctypes.c_int64 * 3), ("v_strides", ctypes.c_int64 * 3),
        ("q_out", ctypes.c_void_p), ("k_out", ctypes.c_void_p), ("v_out", ctypes.c_void_p),
        ("q_weight", ctypes.c_void_p), ("k_weight", ctypes.c_void_p),
        ("cos", ctypes.c_void_p), ("sin", ctypes.c_void_p), ("kv_len", ctypes.c_void_p),
        ("norms", ctypes.c_void_p), ("mk_out", ctypes.c_void_p),
        ("eps", ctypes.c_float), ("scale", ctypes.c_float), ("gate", ctypes.c_float),
        ("B", ctypes.c_int32), ("S", ctypes.c_int32), ("H", ctypes.c_int32), ("D", ctypes.c_int32),
        ("rotary", ctypes.c_int32),
    ]


class SmoothKParams(ctypes.Structure):
    """Mirror of ``dtb_smooth_k_params``."""

    _fields_ = [
        ("k", ctypes.c_void_p),
        ("k_stride_b", ctypes.c_int64), ("k_stride_h", ctypes.c_int64), ("k_stride_s", ctypes.c_int64),
        ("out", ctypes.c_void_p),
        ("out_stride_b", ctypes.c_int64), ("out_stride_h", ctypes.c_int64), ("out_stride_s", ctypes.c_int64),
        ("kv_len", ctypes.c_void_p), ("scratch", ctypes.c_void_p), ("scratch_bytes", ctypes.c_size_t),
        ("k_norm_max", ctypes.c_void_p),
        ("B", ctypes.c_int32), ("H", ctypes.c_int32), ("S", ctypes.c_int32), ("D", ctypes.c_int32),
    ]


class LaunchPlan(ctypes.Structure):
    """Mirror of ``dtb_launch_plan``."""

    _fields_ = [
        ("units", ctypes.c_int32), ("key_tiles", ctypes.c_int32), ("whole_units", ctypes.c_int32),
        ("tail_units", ctypes.c_int32), ("n_pieces", ctypes.c_int32), ("n_slots", ctypes.c_int32),
        ("unit", ctypes.c_int32 * 304), ("tile_begin", ctypes.c_uint16 * 304), ("tile_end", ctypes.c_uint16 * 304),
        ("slot", ctypes.c_int16 * 304),
    ]


class OutProjParams(ctypes.Structure):
    """Mirror of ``dtb_out_proj_params``."""

    _fields_ = [
        ("o", ctypes.c_void_p),
        ("o_stride_b", ctypes.c_int64), ("o_stride_h", ctypes.c_int64), ("o_stride_s", ctypes.c_int64),
        ("w", ctypes.c_void_p), ("w_stride_k", ctypes.c_int64),
        ("out", ctypes.c_void_p), ("out_stride_b", ctypes.c_int64), ("out_stride_s", ctypes.c_int64),
        ("red_dst", ctypes.c_void_p * 8), ("n_dest", ctypes.c_int32), ("rows_per_dest", ctypes.c_int32),
        ("partials", ctypes.c_int32), ("src_rank", ctypes.c_int32),
        ("B", ctypes.c_int32), ("H_local", ctypes.c_int32), ("S", ctypes.c_int32), ("D", ctypes.c_int32),
        ("N", ctypes.c_int32), ("status", ctypes.c_void_p),
    ]


_lock = threading.Lock()
_lib = None


def lib_path() -> str:
    return _build.LIB_PATH


def load(build_if_missing: bool = True) -> ctypes.CDLL:
    """Loads (building first if the binary is absent) and returns the shared library."""
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = os.environ.get("DTB200_LIB") or _build.LIB_PATH   # DTB200_LIB selects another build of the library
        if not os.path.exists(path):
            if not build_if_missing:
                raise RuntimeError(f"{path} is missing; run `python -m dtb200.build`")
            _build.build()
        lib = ctypes.CDLL(path)
        vp, i32p = ctypes.c_void_p, ctypes.c_void_p
        lib.dtb_version.restype = ctypes.c_int
        lib.dtb_status_string.restype = ctypes.c_char_p
        lib.dtb_status_string.argtypes = [ctypes.c_int]
        lib.dtb_last_error_detail.restype = ctypes.c_char_p
        lib.dtb_attn_supported.restype = ctypes.c_int
        lib.dtb_attn_supported.argtypes = [ctypes.POINTER(AttnParams), ctypes.POINTER(ctypes.c_int)]
        lib.dtb_attn_workspace_bytes.restype = ctypes.c_size_t
        lib.dtb_attn_workspace_bytes.argtypes = [ctypes.POINTER(AttnParams)]
        lib.dtb_attn_fwd.restype = ctypes.c_int
        lib.dtb_attn_fwd.argtypes = [ctypes.POINTER(AttnParams), vp, ctypes.c_size_t, vp]
        lib.dtb_attn_launch_plan.restype = ctypes.c_int
        lib.dtb_attn_launch_plan.argtypes = [ctypes.POINTER(AttnParams), ctypes.c_int32, ctypes.POINTER(LaunchPlan)]
        lib.dtb_attn_fwd_static_scratch.restype = ctypes.c_int
        lib.dtb_attn_fwd_static_scratch.argtypes = [ctypes.POINTER(AttnParams), vp]
        lib.dtb_attn_fwd_sparse.restype = ctypes.c_int
        lib.dtb_attn_fwd_sparse.argtypes = [ctypes.POINTER(AttnParams), ctypes.POINTER(BlockTable), vp]
        lib.dtb_quantize_e4m3.restype = ctypes.c_int
        lib.dtb_quantize_e4m3.argtypes = [vp, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int32, ctypes.c_int32,
                                          ctypes.c_int32, ctypes.c_int32, ctypes.c_float, vp, vp]
        lib.dtb_smooth_k.restype = ctypes.c_int
        lib.dtb_smooth_k.argtypes = [ctypes.POINTER(SmoothKParams), vp]
        lib.dtb_smooth_k_scratch_bytes.restype = ctypes.c_size_t
        lib.dtb_smooth_k_scratch_bytes.argtypes = [ctypes.c_int32, ctypes.c_int32]
        lib.dtb_fixed_m_from_norms.restype = ctypes.c_int
        lib.dtb_fixed_m_from_norms.argtypes = [vp, vp, ctypes.c_int32, ctypes.c_int32, ctypes.c_float, vp, vp]
        lib.dtb_sum_partials.restype = ctypes.c_int
        lib.dtb_sum_partials.argtypes = [vp, ctypes.c_int32, ctypes.c_int64, ctypes.c_int32, vp, vp]
        lib.dtb_out_proj.restype = ctypes.c_int
        lib.dtb_out_proj.argtypes = [ctypes.POINTER(OutProjParams), vp]
        lib.dtb_qk_prepass.restype = ctypes.c_int
        lib.dtb_qk_prepass.argtypes = [ctypes.POINTER(PrepassParams), vp]
        lib.dtb_attn_fwd_scatter.restype = ctypes.c_int
        lib.dtb_attn_fwd_scatter.argtypes = [ctypes.POINTER(AttnParams), ctypes.POINTER(AttnScatter), vp]
        lib.dtb_scatter_heads.restype = ctypes.c_int
        lib.dtb_scatter_heads.argtypes = [ctypes.POINTER(ScatterHeadsParams), vp]
        lib.dtb_attn_fwd_residual.restype = ctypes.c_int
        lib.dtb_attn_fwd_residual.argtypes = [ctypes.POINTER(AttnParams), ctypes.POINTER(AttnResidual), vp]
        lib.dtb_attn_finalize.restype = ctypes.c_int
        lib.dtb_attn_finalize.argtypes = [ctypes.POINTER(AttnParams), ctypes.POINTER(AttnResidual), vp]
        lib.dtb_fixed_m_operands.restype = ctypes.c_int
        lib.dtb_fixed_m_operands.argtypes = [ctypes.POINTER(AttnParams), ctypes.c_float, vp, vp, vp]
        for name in ("dtb_selftest_tmem_roundtrip",):
            fn = getattr(lib, name)
            fn.restype = ctypes.c_int
            fn.argtypes = [vp, vp, i32p, vp]
        for name in ("dtb_selftest_qk", "dtb_selftest_pv"):
            fn = getattr(lib, name)
            fn.restype = ctypes.c_int
            fn.argtypes = [vp, vp, vp, i32p, vp]
        lib.dtb_selftest_wait_timeout.restype = ctypes.c_int
        lib.dtb_selftest_wait_timeout.argtypes = [ctypes.c_ulonglong, ctypes.c_int, i32p, i32p, vp]
        _lib = lib
        return lib


def status_string(code: int) -> str:
    return load().dtb_status_string(int(code)).decode()


def check(code: int, what: str) -> None:
    """Maps a C-ABI status to the exception the reference's Python API would raise."""
    if code == DTB_OK:
        return
    msg = f"{what}: {STATUS_NAMES.get(code, code)} ({status_string(code)})"
    detail = load().dtb_last_error_detail().decode()
    if code == 7 and detail:
        msg += f" [{detail}]"
    if code in (2, 3, 9):
        raise NotImplementedError(msg)
    if code in (1, 4, 6):
        raise ValueError(msg)
    raise RuntimeError(msg)
