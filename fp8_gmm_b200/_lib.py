"""ctypes binding of libfp8gmm_b200.so, the C-ABI library declared in include/fp8_gmm_b200.h.

There is no fallback of any kind: if the shared library is missing, importing this module raises, and
every wrapper turns a non-zero status into a RuntimeError carrying the library's error string (the
reference surfaces its TORCH_CHECK failures as RuntimeError too, e.g. reference csrc/fp8_gmm.cu:165-198).
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# FP8GMM_LIBRARY selects another build of the same library (e.g. one compiled with experimental tile sizes)
LIB_PATH = os.environ.get("FP8GMM_LIBRARY") or os.path.join(_HERE, "libfp8gmm_b200.so")

c_i64 = ctypes.c_int64
c_vp = ctypes.c_void_p
c_fp = ctypes.c_void_p  # device float pointers are passed as raw addresses


class TensorDesc(ctypes.Structure):
    _fields_ = [
        ("in_", c_vp), ("in2", c_vp), ("out", c_vp), ("out_t", c_vp), ("scale", c_fp), ("amax", c_fp),
        ("rows", c_i64), ("cols", c_i64), ("padded_rows", c_i64),
    ]


class ScaleMulDesc(ctypes.Structure):
    _fields_ = [("data", c_vp), ("scale1", c_fp), ("scale2", c_fp), ("numel", c_i64)]


class GroupedCastArgs(ctypes.Structure):
    _fields_ = [
        ("in_", c_vp), ("in2", c_vp), ("out", c_vp), ("out_t", c_vp),
        ("row_offsets", ctypes.POINTER(c_i64)), ("t_offsets", ctypes.POINTER(c_i64)),
        ("num_groups", ctypes.c_int), ("cols", c_i64),
        ("scale", c_fp), ("scale_stride", c_i64), ("amax", c_fp), ("amax_stride", c_i64),
        ("out_format", ctypes.c_int), ("activation", ctypes.c_int), ("in_is_fp8", ctypes.c_int),
    ]


class GemmArgs(ctypes.Structure):
    _fields_ = [
        ("a", c_vp), ("b", c_vp), ("c", c_vp), ("m_sizes", ctypes.POINTER(c_i64)),
        ("num_groups", ctypes.c_int), ("n", c_i64), ("k", c_i64),
        ("a_format", ctypes.c_int), ("b_format", ctypes.c_int),
        ("a_scale_inv", c_fp), ("a_scale_inv_stride", c_i64),
        ("b_scale_inv", c_fp), ("b_scale_inv_stride", c_i64),
        ("activation", ctypes.c_int), ("act_out", c_vp),
        ("act_scale", c_fp), ("act_scale_stride", c_i64),
        ("act_amax", c_fp), ("act_amax_stride", c_i64),
        ("c_row_map", c_vp), ("b_layout", ctypes.c_int),
        ("aux_in", c_vp), ("act_out_format", ctypes.c_int),
        ("c_peers", c_vp),
    ]


class BlockedCastArgs(ctypes.Structure):
    _fields_ = [
        ("in_", c_vp), ("out", c_vp),
        ("src_start", ctypes.POINTER(c_i64)), ("dst_start", ctypes.POINTER(c_i64)),
        ("rows", ctypes.POINTER(c_i64)), ("group", ctypes.POINTER(c_i64)),
        ("num_blocks", c_i64), ("cols", c_i64),
        ("scale", c_fp), ("scale_stride", c_i64), ("amax", c_fp), ("amax_stride", c_i64),
        ("out_format", ctypes.c_int),
    ]


class WgradArgs(ctypes.Structure):
    _fields_ = [
        ("a_t", c_vp), ("b_t", c_vp), ("c", c_vp), ("t_offsets", ctypes.POINTER(c_i64)),
        ("num_groups", ctypes.c_int), ("n", c_i64), ("k", c_i64),
        ("a_format", ctypes.c_int), ("b_format", ctypes.c_int),
        ("a_scale_inv", c_fp), ("a_scale_inv_stride", c_i64),
        ("b_scale_inv", c_fp), ("b_scale_inv_stride", c_i64),
        ("workspace", c_vp), ("workspace_bytes", ctypes.c_size_t),
    ]


class CopyBlock(ctypes.Structure):
    _fields_ = [("dst", c_vp), ("src", c_vp), ("bytes", ctypes.c_size_t)]


# name -> (restype, argtypes); must list every symbol the header declares (tests/test_abi.py checks).
SYMBOLS = {
    "fp8gmm_version": (ctypes.c_int, []),
    "fp8gmm_last_error": (ctypes.c_char_p, []),
    "fp8gmm_device_status": (ctypes.c_int, [c_vp]),
    "fp8gmm_launch_count": (ctypes.c_uint64, []),
    "fp8gmm_multi_quantize": (ctypes.c_int, [ctypes.POINTER(TensorDesc), ctypes.c_int, ctypes.c_int, c_vp]),
    "fp8gmm_multi_pad_transpose": (ctypes.c_int, [ctypes.POINTER(TensorDesc), ctypes.c_int, c_vp]),
    "fp8gmm_multi_pad_cast_transpose": (ctypes.c_int, [ctypes.POINTER(TensorDesc), ctypes.c_int, ctypes.c_int, c_vp]),
    "fp8gmm_multi_pad_cast_transpose_dgelu": (ctypes.c_int, [ctypes.POINTER(TensorDesc), ctypes.c_int, ctypes.c_int, c_vp]),
    "fp8gmm_multi_pad_cast_transpose_dswiglu": (ctypes.c_int, [ctypes.POINTER(TensorDesc), ctypes.c_int, ctypes.c_int, c_vp]),
    "fp8gmm_multi_scale_mul": (ctypes.c_int, [ctypes.POINTER(ScaleMulDesc), ctypes.c_int, c_vp]),
    "fp8gmm_grouped_pad_cast_transpose": (ctypes.c_int, [ctypes.POINTER(GroupedCastArgs), c_vp]),
    "fp8gmm_blocked_cast": (ctypes.c_int, [ctypes.POINTER(BlockedCastArgs), c_vp]),
    "fp8gmm_grouped_gemm": (ctypes.c_int, [ctypes.POINTER(GemmArgs), c_vp]),
    "fp8gmm_wgrad_workspace_bytes": (ctypes.c_size_t, [ctypes.c_int]),
    "fp8gmm_grouped_wgrad": (ctypes.c_int, [ctypes.POINTER(WgradArgs), c_vp]),
    "fp8gmm_grouped_wgrad_static": (ctypes.c_int, [ctypes.POINTER(WgradArgs), c_vp]),
    "fp8gmm_grouped_wgrad_rowmajor": (ctypes.c_int, [ctypes.POINTER(WgradArgs), c_vp]),
    "fp8gmm_set_gemm_sm_limit": (ctypes.c_int, [ctypes.c_int]),
    "fp8gmm_set_gemm_variant": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, ctypes.c_int]),
    "fp8gmm_device_status_async": (ctypes.c_int, [c_vp, c_vp]),
    "fp8gmm_set_wait_limits": (ctypes.c_int, [c_i64, c_i64]),
    "fp8gmm_moe_topk": (ctypes.c_int, [c_vp, ctypes.c_int, c_i64, ctypes.c_int, ctypes.c_int, ctypes.c_int, c_vp, c_vp, c_vp, c_vp]),
    "fp8gmm_moe_sort": (ctypes.c_int, [c_vp, c_i64, ctypes.c_int, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp]),
    "fp8gmm_moe_gather": (ctypes.c_int, [c_vp, c_vp, c_vp, ctypes.c_int, c_i64, c_i64, c_vp, c_vp]),
    "fp8gmm_moe_scatter": (ctypes.c_int, [c_vp, c_vp, c_vp, ctypes.c_int, c_i64, c_i64, c_vp, c_vp]),
    "fp8gmm_moe_rowdot": (ctypes.c_int, [c_vp, c_vp, c_vp, ctypes.c_int, c_i64, c_i64, c_vp, c_vp]),
    "fp8gmm_peer_alloc": (ctypes.c_int, [ctypes.c_size_t, ctypes.POINTER(c_vp), c_vp]),
    "fp8gmm_peer_free": (ctypes.c_int, [c_vp]),
    "fp8gmm_peer_open": (ctypes.c_int, [c_vp, ctypes.POINTER(c_vp)]),
    "fp8gmm_peer_close": (ctypes.c_int, [c_vp]),
    "fp8gmm_peer_copy_blocks": (ctypes.c_int, [ctypes.POINTER(CopyBlock), ctypes.c_int, c_vp]),
    "fp8gmm_block_permute_rows": (ctypes.c_int, [c_vp, c_vp, ctypes.POINTER(c_i64), ctypes.POINTER(c_i64), ctypes.POINTER(c_i64), c_i64, c_i64, c_vp]),
    "fp8gmm_peer_signal": (ctypes.c_int, [ctypes.POINTER(c_vp), ctypes.c_int, ctypes.c_uint32, c_vp]),
    "fp8gmm_peer_wait": (ctypes.c_int, [c_vp, ctypes.c_int, ctypes.c_uint32, c_vp]),
    "fp8gmm_peer_reduce_scatter_bf16": (ctypes.c_int, [ctypes.POINTER(c_vp), ctypes.c_int, ctypes.c_int, c_i64, c_i64, ctypes.c_int, c_vp]),
    "fp8gmm_peer_all_gather_bf16": (ctypes.c_int, [ctypes.POINTER(c_vp), ctypes.c_int, ctypes.c_int, c_i64, c_i64, c_vp, ctypes.c_int, c_vp]),
    "fp8gmm_delayed_scaling_update": (
        ctypes.c_int,
        [c_fp, c_fp, c_fp, ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_float, ctypes.c_int, c_vp],
    ),
}

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python fp8_gmm_b200/csrc/build.py` (needs nvcc). "
        "fp8_gmm_b200 has no CPU or PyTorch fallback."
    )

lib = ctypes.CDLL(LIB_PATH)
for _name, (_res, _args) in SYMBOLS.items():
    try:
        _fn = getattr(lib, _name)
    except AttributeError as exc:
        raise ImportError(
            f"{LIB_PATH} does not export {_name}: it is older than the sources; rebuild it with "
            "`python fp8_gmm_b200/csrc/build.py`"
        ) from exc
    _fn.restype = _res
    _fn.argtypes = _args


def check(status, what):
    """Raise RuntimeError for a non-zero status, like the reference's TORCH_CHECK failures."""
    if status != 0:
        msg = lib.fp8gmm_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"fp8_gmm_b200.{what} failed (status {status}): {msg}")
