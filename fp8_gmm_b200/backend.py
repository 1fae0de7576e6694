"""Backend ops with the names, argument order and error behaviour of the reference's fp8_gmm/backend.py.

Every function enqueues hand-written sm_100a kernels through the C ABI (include/fp8_gmm_b200.h) on
torch's current CUDA stream and returns without synchronising.  Outputs are caller-allocated and
written in place, exactly like the reference's pybind ops (reference csrc/ops.cu:9-16).  Contract
violations raise RuntimeError (the reference raises it from TORCH_CHECK).  There is no CPU path.

List-style ops accept any number of tensors per call (the reference stops at 64).  The ``grouped_*``
functions are the allocation-free fast forms the modules use: one base tensor plus host prefix sums
instead of Python lists of per-group views.
"""
import ctypes
import os

import numpy as np
import torch

from . import _lib
from ._lib import BlockedCastArgs, GemmArgs, GroupedCastArgs, ScaleMulDesc, TensorDesc, WgradArgs, check, lib
from .utils import FP8_FORMAT_CODE

_FP8 = (torch.float8_e4m3fn, torch.float8_e5m2)
# Weight gradients read the row-major FP8 activations directly (grouped_wgrad_rowmajor), so the modules make no
# padded-transposed copies.  FP8GMM_WGRAD=transposed selects the reference's dataflow instead (padded transposes
# written by the cast kernels, reference fp8_gmm/grouped_linear.py:32-52,133-149, consumed by grouped_wgrad).
WGRAD_ROWMAJOR = os.environ.get("FP8GMM_WGRAD", "rowmajor") != "transposed"
# Data gradients multiply by the forward FP8 weights (G, out, in) as they are (fp8_gmm(..., b_is_kn=True)), so the
# modules make no per-expert weight transposes either.  FP8GMM_DGRAD=transposed selects the reference's dataflow
# (weights cast into (G, in, out) transposes, reference fp8_gmm/grouped_linear.py:70-73).
DGRAD_KN = os.environ.get("FP8GMM_DGRAD", "kn") != "transposed"
# FP8GMM_FUSED_DSWIGLU=1 runs the SwiGLU backward in the epilogue of the fc2 data-gradient GEMM (fp8_gmm_dswiglu) whenever
# no transposed copy of its result is wanted.  Off by default: on the Mixtral-shaped step the fused epilogue (one row
# per thread, so its pre-activation loads do not coalesce) stretches that GEMM by more than the separate
# activation-backward kernel costs (16.67-16.71 against 16.28-16.61 ms per step).
FUSED_DSWIGLU = os.environ.get("FP8GMM_FUSED_DSWIGLU", "0") == "1"
ACT_NONE, ACT_GELU, ACT_SWIGLU, ACT_DSWIGLU = 0, 1, 2, 3
_ACT_CODE = {None: 0, "none": 0, "gelu": 1, "swiglu": 2}


try:  # the raw getters skip torch.cuda.current_stream()'s object construction (about 20 us per call, per launch)
    _raw_stream, _raw_device = torch._C._cuda_getCurrentRawStream, torch._C._cuda_getDevice
except AttributeError:  # pragma: no cover - other torch builds
    _raw_stream = _raw_device = None


def _stream():
    """cudaStream_t of torch's current stream on the current device, as an integer."""
    if _raw_stream is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


# Optional per-launch timing of the GEMM kernel (used by bench.py for its roofline line): when a list is
# installed, every GEMM call appends (start_event, end_event, flops) recorded on the launching stream.
_gemm_timings = None


def set_gemm_timings(sink):
    """Install (or with None remove) a list that receives (start, end, flops) per GEMM launch."""
    global _gemm_timings
    _gemm_timings = sink


def set_gemm_sm_limit(sms):
    """Cap the SMs the persistent GEMM kernels occupy (0 = all); see fp8gmm_set_gemm_sm_limit."""
    check(lib.fp8gmm_set_gemm_sm_limit(int(sms)), "set_gemm_sm_limit")


def set_gemm_variant(ctas=0, tail_split=True, tma_epilogue=True):
    """Force the GEMM tile shape (1 = single-CTA 128-row tiles, 2 = CTA-pair 256-row tiles, 0 = automatic) and the
    two launch switches; see fp8gmm_set_gemm_variant.  For tests and experiments: results are bit-identical."""
    check(lib.fp8gmm_set_gemm_variant(int(ctas), int(bool(tail_split)), int(bool(tma_epilogue))), "set_gemm_variant")


def set_wait_limits(gemm_wait_s=0.0, peer_wait_s=0.0):
    """Limits of the kernels' bounded waits in seconds (0 keeps the current value); see fp8gmm_set_wait_limits."""
    check(lib.fp8gmm_set_wait_limits(int(gemm_wait_s * 1e9), int(peer_wait_s * 1e9)), "set_wait_limits")


def launch_count():
    """Kernels launched by the C-ABI library in this process so far."""
    return int(lib.fp8gmm_launch_count())


class _Timed:
    def __init__(self, flops):
        self.flops = flops

    def __enter__(self):
        if _gemm_timings is not None:
            self.start = torch.cuda.Event(enable_timing=True)
            self.start.record()

    def __exit__(self, *exc):
        if _gemm_timings is not None:
            end = torch.cuda.Event(enable_timing=True)
            end.record()
            _gemm_timings.append((self.start, end, self.flops))


def _require(cond, msg):
    if not cond:
        raise RuntimeError(msg)


def _ptr(t):
    return None if t is None else t.data_ptr()


def _i64_array(values):
    """Host int64 array for the C ABI from a CPU int64 tensor (zero copy) or any int sequence."""
    if torch.is_tensor(values):
        _require(values.device.type == "cpu", "group sizes / offsets must be a CPU tensor")
        t = values.to(torch.int64).contiguous()
        return ctypes.cast(t.data_ptr(), ctypes.POINTER(ctypes.c_int64)), t
    arr = np.asarray(values, dtype=np.int64)
    return ctypes.cast(arr.ctypes.data, ctypes.POINTER(ctypes.c_int64)), arr


def _fp8_code(dtype):
    _require(dtype in _FP8, f"expected a float8 dtype, got {dtype}")
    return FP8_FORMAT_CODE[dtype]


def _cuda_2d(t, name, dtypes):
    _require(t.is_cuda, f"{name} must be a CUDA tensor")
    _require(t.dtype in dtypes, f"{name} has dtype {t.dtype}, expected one of {dtypes}")
    _require(t.is_contiguous(), f"{name} must be contiguous")


class _Strided:
    """Per-group fp32 slots addressed as base[g * stride] on the device."""

    __slots__ = ("ptr", "stride", "keep", "scatter")

    def __init__(self, ptr, stride, keep=None, scatter=None):
        self.ptr, self.stride, self.keep, self.scatter = ptr, stride, keep, scatter


def _strided(spec, count, writable=False):
    """Accepts None, a (tensor, stride) pair, one tensor with `count` elements, or a list of 0-dim /
    1-element tensors (the reference's form).  Lists whose elements are not evenly spaced in memory
    are gathered into a temporary (and scattered back afterwards when ``writable``)."""
    if spec is None:
        return _Strided(None, 0)
    if isinstance(spec, tuple):
        t, stride = spec
        _require(t.is_cuda and t.dtype == torch.float32, "meta tensors must be CUDA float32")
        return _Strided(t.data_ptr(), int(stride) * t.stride(0) if t.dim() else 0, keep=t)
    if torch.is_tensor(spec):
        _require(spec.is_cuda and spec.dtype == torch.float32, "meta tensors must be CUDA float32")
        _require(spec.numel() >= count, "meta tensor has fewer elements than groups")
        flat = spec.reshape(-1)
        return _Strided(flat.data_ptr(), flat.stride(0) if flat.numel() > 1 else 0, keep=flat)
    items = list(spec)
    _require(len(items) == count, f"expected {count} per-group meta tensors, got {len(items)}")
    for t in items:
        _require(t.is_cuda and t.dtype == torch.float32 and t.numel() == 1, "meta tensors must be CUDA float32 scalars")
    if count == 0:
        return _Strided(None, 0)
    p0 = items[0].data_ptr()
    if count == 1:
        return _Strided(p0, 0, keep=items)
    step = items[1].data_ptr() - p0
    if step % 4 == 0 and all(items[i].data_ptr() - p0 == i * step for i in range(count)):
        return _Strided(p0, step // 4, keep=items)
    packed = torch.stack([t.reshape(()) for t in items])
    scatter = (lambda: [t.copy_(packed[i].reshape(t.shape)) for i, t in enumerate(items)]) if writable else None
    return _Strided(packed.data_ptr(), 1, keep=packed, scatter=scatter)


# ------------------------------------------------------------------------------------------------
# multi-tensor elementwise ops (reference fp8_gmm/backend.py:9-22)
# ------------------------------------------------------------------------------------------------
def _descs(inputs, in2s, outputs, trans_outputs, scales, amaxes, in_dtypes, wide_out=1):
    n = len(inputs)
    arr = (TensorDesc * max(n, 1))()
    for i in range(n):
        x = inputs[i]
        _cuda_2d(x, f"inputs[{i}]", in_dtypes)
        rows, cols = (x.shape[0], x.shape[1]) if x.dim() == 2 else (1, x.numel()) if x.dim() <= 1 else (
            x.numel() // x.shape[-1], x.shape[-1])
        d = arr[i]
        d.in_ = x.data_ptr()
        d.rows, d.cols, d.padded_rows = rows, cols, rows
        if in2s is not None:
            g = in2s[i]
            _cuda_2d(g, f"second inputs[{i}]", (torch.bfloat16,))
            _require(g.numel() == x.numel() * wide_out, f"second inputs[{i}] has the wrong size")
            d.in2 = g.data_ptr()
        if outputs is not None:
            o = outputs[i]
            _cuda_2d(o, f"outputs[{i}]", _FP8)
            _require(o.numel() == x.numel() * wide_out, f"outputs[{i}] does not match the shape of its input")
            d.out = o.data_ptr()
        if trans_outputs is not None:
            t = trans_outputs[i]
            _cuda_2d(t, f"trans_outputs[{i}]", _FP8)
            _require(t.dim() == 2 and t.shape[0] == cols * wide_out and t.shape[1] >= rows,
                     f"trans_outputs[{i}] must have shape ({cols * wide_out}, >= {rows}), got {tuple(t.shape)}")
            d.out_t = t.data_ptr()
            d.padded_rows = t.shape[1]
        if scales is not None and scales[i] is not None:
            _require(scales[i].is_cuda and scales[i].dtype == torch.float32, "scales must be CUDA float32")
            d.scale = scales[i].data_ptr()
        if amaxes is not None and amaxes[i] is not None:
            _require(amaxes[i].is_cuda and amaxes[i].dtype == torch.float32, "amaxes must be CUDA float32")
            d.amax = amaxes[i].data_ptr()
    return arr, n


def _same_len(*lists):
    n = len(lists[0])
    for l in lists[1:]:
        _require(l is None or len(l) == n, "tensor lists must have the same length")


def multi_quantize(inputs, outputs, scales, amaxes):
    """bf16 -> fp8 ``OType(scale * x)`` + amax for every tensor (reference fp8_gmm/backend.py:9-10)."""
    if len(inputs) == 0:
        return
    _same_len(inputs, outputs, scales, amaxes)
    arr, n = _descs(inputs, None, outputs, None, scales, amaxes, (torch.bfloat16,))
    check(lib.fp8gmm_multi_quantize(arr, n, _fp8_code(outputs[0].dtype), _stream()), "multi_quantize")


def multi_amax(inputs, amaxes):
    """amax only (no FP8 output): first pass of per-tensor current scaling."""
    if len(inputs) == 0:
        return
    _same_len(inputs, amaxes)
    arr, n = _descs(inputs, None, None, None, None, amaxes, (torch.bfloat16,))
    check(lib.fp8gmm_multi_quantize(arr, n, 0, _stream()), "multi_amax")


def multi_transpose(inputs, outputs):
    """fp8 (m, n) -> fp8 (n, M >= m), zero padded (reference fp8_gmm/backend.py:13-14)."""
    if len(inputs) == 0:
        return
    _same_len(inputs, outputs)
    for x, o in zip(inputs, outputs):
        _require(x.dtype == o.dtype, "multi_transpose: input and output dtypes differ")
    arr, n = _descs(inputs, None, None, outputs, None, None, _FP8)
    check(lib.fp8gmm_multi_pad_transpose(arr, n, _stream()), "multi_transpose")


def multi_cast_transpose(inputs, outputs, trans_outputs, scales, amaxes):
    """bf16 -> fp8 cast + padded transpose + amax (reference fp8_gmm/backend.py:17-18)."""
    if len(inputs) == 0:
        return
    _same_len(inputs, outputs, trans_outputs, scales, amaxes)
    arr, n = _descs(inputs, None, outputs, trans_outputs, scales, amaxes, (torch.bfloat16,))
    check(lib.fp8gmm_multi_pad_cast_transpose(arr, n, _fp8_code(outputs[0].dtype), _stream()), "multi_cast_transpose")


def multi_cast_transpose_dgelu(inputs, gelu_inputs, outputs, trans_outputs, scales, amaxes):
    """As multi_cast_transpose on ``inputs * dgelu(gelu_inputs)`` (reference fp8_gmm/backend.py:21-22)."""
    if len(inputs) == 0:
        return
    _same_len(inputs, gelu_inputs, outputs, trans_outputs, scales, amaxes)
    arr, n = _descs(inputs, gelu_inputs, outputs, trans_outputs, scales, amaxes, (torch.bfloat16,))
    check(lib.fp8gmm_multi_pad_cast_transpose_dgelu(arr, n, _fp8_code(outputs[0].dtype), _stream()),
          "multi_cast_transpose_dgelu")


def multi_cast_transpose_dswiglu(inputs, swiglu_inputs, outputs, trans_outputs, scales, amaxes):
    """SwiGLU backward fused with the cast: inputs (m, F) = d(act), swiglu_inputs (m, 2F) = [gate | up];
    outputs (m, 2F) and trans_outputs (2F, M).  Extension beyond the reference (GELU only there)."""
    if len(inputs) == 0:
        return
    _same_len(inputs, swiglu_inputs, outputs, trans_outputs, scales, amaxes)
    arr, n = _descs(inputs, swiglu_inputs, outputs, trans_outputs, scales, amaxes, (torch.bfloat16,), wide_out=2)
    check(lib.fp8gmm_multi_pad_cast_transpose_dswiglu(arr, n, _fp8_code(outputs[0].dtype), _stream()),
          "multi_cast_transpose_dswiglu")


def multi_scale_mul(inputs, scales_1, scales_2):
    """In place ``x = bf16(fp32(x) * s1 * s2)`` (the reference's backend.multi_scale_mul, csrc/ops.cu:12)."""
    if len(inputs) == 0:
        return
    _same_len(inputs, scales_1, scales_2)
    n = len(inputs)
    arr = (ScaleMulDesc * n)()
    for i, x in enumerate(inputs):
        _cuda_2d(x, f"inputs[{i}]", (torch.bfloat16,))
        arr[i].data = x.data_ptr()
        arr[i].scale1 = _ptr(scales_1[i])
        arr[i].scale2 = _ptr(scales_2[i])
        arr[i].numel = x.numel()
    check(lib.fp8gmm_multi_scale_mul(arr, n, _stream()), "multi_scale_mul")


def grouped_cast_transpose(inp, row_offsets, out, out_t, t_offsets, scale, amax, in2=None, activation=None):
    """Grouped form of the cast/transposes: ``inp`` is one (sum rows, cols) matrix whose row blocks are the
    groups; see fp8gmm_grouped_pad_cast_transpose in the header.  ``scale`` / ``amax`` are
    (tensor, stride) pairs.  An fp8 ``inp`` makes it a pure padded transpose."""
    G = len(row_offsets) - 1
    args = GroupedCastArgs()
    in_is_fp8 = inp.dtype in _FP8
    _cuda_2d(inp, "inp", _FP8 if in_is_fp8 else (torch.bfloat16,))
    args.in_ = inp.data_ptr()
    args.in2 = _ptr(in2)
    args.out = _ptr(out)
    args.out_t = _ptr(out_t)
    ro, keep1 = _i64_array(row_offsets)
    args.row_offsets = ro
    keep2 = None
    if out_t is not None:
        to, keep2 = _i64_array(t_offsets)
        args.t_offsets = to
    args.num_groups = G
    args.cols = inp.shape[1]
    s = _strided(scale, G)
    a = _strided(amax, G, writable=True)
    args.scale, args.scale_stride = s.ptr, s.stride
    args.amax, args.amax_stride = a.ptr, a.stride
    ref_out = out if out is not None else out_t
    args.out_format = _fp8_code(ref_out.dtype)
    args.activation = _ACT_CODE[activation]
    args.in_is_fp8 = int(in_is_fp8)
    check(lib.fp8gmm_grouped_pad_cast_transpose(ctypes.byref(args), _stream()), "grouped_cast_transpose")
    if a.scatter:
        a.scatter()
    del keep1, keep2


# ------------------------------------------------------------------------------------------------
# GEMMs (reference fp8_gmm/backend.py:25-97)
# ------------------------------------------------------------------------------------------------
class RowPermutation:
    """Block permutation between an external row order and the expert-major order the grouped kernels use.

    Block b is ``rows[b]`` consecutive rows that sit at external row ``src_start[b]`` and belong at expert-major
    row ``dst_start[b]`` of group ``group[b]`` (host int64 sequences).  ``row_map`` is the same permutation per
    row as a device int32 tensor: expert-major row r <-> external row row_map[r].  Used by expert parallelism,
    where the all-to-all delivers rows source-major."""

    def __init__(self, src_start, dst_start, rows, group, row_map):
        self.num_blocks = len(rows)
        self._keep = [_i64_array(v) for v in (src_start, dst_start, rows, group)]
        self.src_start, self.dst_start, self.rows, self.group = [k[0] for k in self._keep]
        self.row_map = row_map
        assert row_map.dtype == torch.int32 and row_map.is_cuda and row_map.is_contiguous()


def blocked_cast(inp, out, perm, scale, amax, num_groups):
    """bf16 rows in external order -> fp8 rows in expert-major order (+ per-group amax); see fp8gmm_blocked_cast."""
    _cuda_2d(inp, "inp", (torch.bfloat16,))
    _cuda_2d(out, "out", _FP8)
    _require(inp.shape == out.shape, "blocked_cast: shapes differ")
    args = BlockedCastArgs()
    args.in_, args.out = inp.data_ptr(), out.data_ptr()
    args.src_start, args.dst_start, args.rows, args.group = perm.src_start, perm.dst_start, perm.rows, perm.group
    args.num_blocks, args.cols = perm.num_blocks, inp.shape[1]
    s = _strided(scale, num_groups)
    a = _strided(amax, num_groups, writable=True)
    args.scale, args.scale_stride = s.ptr, s.stride
    args.amax, args.amax_stride = a.ptr, a.stride
    args.out_format = _fp8_code(out.dtype)
    check(lib.fp8gmm_blocked_cast(ctypes.byref(args), _stream()), "blocked_cast")
    if a.scatter:
        a.scatter()


def block_permute_rows(src, dst, src_start, dst_start, rows):
    """Block permutation of rows between two tensors of equal row width: block b = ``rows[b]`` consecutive rows from
    row ``src_start[b]`` of ``src`` to row ``dst_start[b]`` of ``dst`` (host int64 sequences); see
    fp8gmm_block_permute_rows."""
    _require(src.is_cuda and dst.is_cuda and src.is_contiguous() and dst.is_contiguous(), "block_permute_rows: contiguous CUDA tensors")
    _require(src.dim() == 2 and dst.dim() == 2 and src.shape[1] == dst.shape[1] and src.dtype == dst.dtype,
             "block_permute_rows: tensors must be 2-D with the same row width and dtype")
    a, k1 = _i64_array(src_start)
    b, k2 = _i64_array(dst_start)
    n, k3 = _i64_array(rows)
    check(lib.fp8gmm_block_permute_rows(src.data_ptr(), dst.data_ptr(), a, b, n, len(rows), src.shape[1] * src.element_size(),
                                        _stream()), "block_permute_rows")
    del k1, k2, k3


def _gemm(a, b3, c, m_sizes, num_groups, sa, sb, activation, act_out, sc, amax, c_row_map=None, b_layout=0, aux_in=None,
          c_peers=None):
    args = GemmArgs()
    args.a, args.b, args.c = a.data_ptr(), b3.data_ptr(), _ptr(c)
    if aux_in is not None:
        args.aux_in, args.act_out_format = aux_in.data_ptr(), _fp8_code(act_out.dtype)
    ms, keep = _i64_array(m_sizes)
    args.m_sizes = ms
    args.num_groups = num_groups
    args.n, args.k = (b3.shape[-2], b3.shape[-1]) if b_layout == 0 else (b3.shape[-1], b3.shape[-2])
    args.b_layout = b_layout
    args.a_format, args.b_format = _fp8_code(a.dtype), _fp8_code(b3.dtype)
    args.a_scale_inv, args.a_scale_inv_stride = sa.ptr, sa.stride
    args.b_scale_inv, args.b_scale_inv_stride = sb.ptr, sb.stride
    args.activation = activation
    args.act_out = _ptr(act_out)
    args.act_scale, args.act_scale_stride = sc.ptr, sc.stride
    args.act_amax, args.act_amax_stride = amax.ptr, amax.stride
    if c_row_map is not None:
        _require(c_row_map.is_cuda and c_row_map.dtype == torch.int32 and c_row_map.numel() == a.shape[0],
                 "c_row_map must be a CUDA int32 tensor with one entry per row of a")
        args.c_row_map = c_row_map.data_ptr()
    if c_peers is not None:
        _require(c_row_map is not None and c_peers.is_cuda and c_peers.dtype == torch.int64 and c_peers.is_contiguous(),
                 "c_peers must be a CUDA int64 tensor of base addresses and needs a c_row_map")
        args.c_peers = c_peers.data_ptr()
    with _Timed(2.0 * a.shape[0] * args.n * args.k):
        check(lib.fp8gmm_grouped_gemm(ctypes.byref(args), _stream()), "fp8_gmm")
    if amax.scatter:
        amax.scatter()
    del keep


ROW_MAP_PEER_SHIFT = 26   # FP8GMM_ROW_MAP_PEER_SHIFT of the C header


def peer_row_entry(rank, row):
    """Row-map entry (works on ints and numpy arrays) naming row ``row`` of rank ``rank``'s buffer (see fp8_gmm, c_peers)."""
    return (rank << ROW_MAP_PEER_SHIFT) | row


def cublas_fp8_gemm(a, b, c, a_scale_inv, b_scale_inv, pre_gelu_out=None, c_scale=None, c_amax=None, backward=False):
    """Single GEMM ``c = (a * a_scale_inv) (b * b_scale_inv)^T`` with a (M, K) and b (N, K) in FP8.

    Same signature as reference fp8_gmm/backend.py:26; the name is kept for drop-in use although the
    work is done by this package's tcgen05 kernel, not cuBLASLt.  With an FP8 ``c`` the GELU-aux
    epilogue is selected: ``pre_gelu_out`` receives the bf16 pre-activation, ``c`` the e4m3 of
    ``gelu(.) * c_scale`` and ``c_amax`` is max-merged with ``max|gelu(.)|``.  ``backward`` selected
    cuBLASLt's split accumulator in the reference; accumulation here is always full fp32.
    """
    _cuda_2d(a, "a", _FP8)
    _cuda_2d(b, "b", _FP8)
    _require(a.dim() == 2 and b.dim() == 2 and a.shape[1] == b.shape[1], "cublas_fp8_gemm: shapes do not contract")
    _require(tuple(c.shape) == (a.shape[0], b.shape[0]) and c.is_contiguous(), "cublas_fp8_gemm: bad output shape")
    sa = _strided([a_scale_inv.reshape(-1)[0:1]], 1)
    sb = _strided([b_scale_inv.reshape(-1)[0:1]], 1)
    m_sizes = [a.shape[0]]
    if c.dtype in _FP8:
        _require(c_scale is not None and c_amax is not None, "cublas_fp8_gemm: FP8 output needs c_scale and c_amax")
        _require(c.dtype == torch.float8_e4m3fn, "cublas_fp8_gemm: FP8 output must be e4m3")
        _require(pre_gelu_out is not None and pre_gelu_out.dtype == torch.bfloat16 and pre_gelu_out.is_contiguous(),
                 "cublas_fp8_gemm: FP8 output needs a bf16 pre_gelu_out")
        _gemm(a, b, pre_gelu_out, m_sizes, 1, sa, sb, ACT_GELU, c, _strided([c_scale.reshape(-1)[0:1]], 1),
              _strided([c_amax.reshape(-1)[0:1]], 1, writable=True))
    else:
        _require(c.dtype == torch.bfloat16, "cublas_fp8_gemm: output must be bfloat16 or float8_e4m3fn")
        _require(pre_gelu_out is None, "cublas_fp8_gemm: pre_gelu_out needs an FP8 output")
        _gemm(a, b, c, m_sizes, 1, sa, sb, ACT_NONE, None, _Strided(None, 0), _Strided(None, 0))


def fp8_gmm(
    a,
    b,
    group_sizes,
    a_scale_invs,
    b_scale_invs,
    c=None,
    c_dtype=torch.bfloat16,
    pre_gelu_out=None,
    c_scales=None,
    c_amaxes=None,
    backward=False,
    cutlass=False,
    activation="gelu",
    c_row_map=None,
    b_is_kn=False,
    c_peers=None,
):
    """Grouped GEMM ``c[rows of g] = (a[rows of g] * sa[g]) (b[g] * sb[g])^T`` in one launch.

    Signature of reference fp8_gmm/backend.py:58-71 plus ``activation``.  a: (sum m, K) FP8 row-major,
    b: (G, N, K) e4m3/e5m2, group_sizes: CPU int64 tensor (or list), scale lists: per-group CUDA fp32
    scalars (lists of 0-dim views as in the reference, a (tensor, stride) pair, or one tensor).
    ``cutlass`` is accepted and ignored: there is a single backend and it fuses the de-scale that the
    reference's CUTLASS path runs as a second pass.  With an FP8 ``c`` (or c_dtype) the fused
    activation epilogue runs: ``pre_gelu_out`` gets the bf16 pre-activation, ``c`` the e4m3
    activation scaled by c_scales[g], c_amaxes[g] the amax.  activation="swiglu" expects b = [gate
    rows | up rows] (N = 2F) and produces a (sum m, F) ``c``.  ``c_row_map`` (CUDA int32, one entry per row
    of a; plain bf16 output only) makes the epilogue store row r of the product at row c_row_map[r] of c.
    ``c_peers`` (CUDA int64: base addresses of one bf16 (rows, N) buffer per rank, peer-mapped) with a ``c_row_map``
    whose entries are ``peer_row_entry(rank, row)``: the epilogue stores every row straight into the named rank's
    buffer (expert parallelism: results leave for their home ranks without a copy); ``c`` must be None, None is returned.
    ``b_is_kn=True``: b is (G, K, N) row-major and ``c = a @ b[g]`` without a transpose -- dgrad with the forward weights
    (G, out, in) as they are (the tensor cores read B MN-major; no per-expert weight transposes needed).
    """
    _cuda_2d(a, "a", _FP8)
    _cuda_2d(b, "b", _FP8)
    _require(a.dim() == 2 and b.dim() == 3, "fp8_gmm: a must be 2-D and b 3-D")
    _require(a.shape[1] == (b.shape[1] if b_is_kn else b.shape[2]), "fp8_gmm: contraction dimensions differ")
    G = b.shape[0]
    _require(len(group_sizes) == G, "fp8_gmm: one group size per expert is required")
    n_out = b.shape[2] if b_is_kn else b.shape[1]
    fused = (c is not None and c.dtype in _FP8) or (c is None and c_dtype in _FP8)
    if fused and activation == "swiglu":
        n_out = b.shape[1] // 2
    if c_peers is not None:
        _require(c is None and not fused and c_row_map is not None, "fp8_gmm: c_peers takes the place of a plain bf16 c")
        sa, sb = _strided(a_scale_invs, G), _strided(b_scale_invs, G)
        _gemm(a, b, None, group_sizes, G, sa, sb, ACT_NONE, None, _Strided(None, 0), _Strided(None, 0), c_row_map,
              b_layout=1 if b_is_kn else 0, c_peers=c_peers)
        return None
    if c is None:
        c = torch.empty(a.shape[0], n_out, device=a.device, dtype=c_dtype)
    _require(tuple(c.shape) == (a.shape[0], n_out) and c.is_contiguous(), "fp8_gmm: bad output shape")
    if cutlass:
        _require(c.dtype == torch.bfloat16 and pre_gelu_out is None, "fp8_gmm: cutlass=True has no fused activation")
    sa = _strided(a_scale_invs, G)
    sb = _strided(b_scale_invs, G)
    _require(not (fused and b_is_kn), "fp8_gmm: b_is_kn has no fused activation")
    if fused:
        _require(c.dtype == torch.float8_e4m3fn, "fp8_gmm: FP8 output must be e4m3")
        _require(c_scales is not None and c_amaxes is not None, "fp8_gmm: FP8 output needs c_scales and c_amaxes")
        _require(pre_gelu_out is not None and pre_gelu_out.dtype == torch.bfloat16 and pre_gelu_out.is_contiguous()
                 and tuple(pre_gelu_out.shape) == (a.shape[0], b.shape[1]), "fp8_gmm: bad pre-activation output")
        _gemm(a, b, pre_gelu_out, group_sizes, G, sa, sb, _ACT_CODE[activation], c, _strided(c_scales, G),
              _strided(c_amaxes, G, writable=True))
    else:
        _require(c.dtype == torch.bfloat16, "fp8_gmm: output must be bfloat16 or float8_e4m3fn")
        _require(pre_gelu_out is None, "fp8_gmm: pre_gelu_out needs an FP8 output")
        _gemm(a, b, c, group_sizes, G, sa, sb, ACT_NONE, None, _Strided(None, 0), _Strided(None, 0), c_row_map,
              b_layout=1 if b_is_kn else 0)
    return c


def fp8_gmm_dswiglu(dy, w, group_sizes, dy_scale_invs, w_scale_invs, pre_act, out, out_scales, out_amaxes, b_is_kn=False):
    """fc2 data gradient with the SwiGLU backward fused in its epilogue, one launch:
    ``d_act = (dy[rows of g] * sa[g]) (w[g] * sb[g])`` (rounded to bf16 as the plain GEMM stores it), then
    ``out[rows of g] = fp8( dswiglu(d_act, pre_act) * out_scales[g] )`` = [d gate | d up] (sum m, 2F) with
    ``out_amaxes[g]`` max-merged.  dy: (sum m, H) FP8; w: (G, F, H) FP8 K-major, or with ``b_is_kn`` the forward fc2
    weights (G, H, F) as they are; pre_act: (sum m, 2F) bf16 = [gate | up].  Replaces fp8_gmm + the dswiglu cast kernel
    (the d_act matrix never goes to memory).  Extension beyond the reference (GELU only there)."""
    _cuda_2d(dy, "dy", _FP8)
    _cuda_2d(w, "w", _FP8)
    _cuda_2d(pre_act, "pre_act", (torch.bfloat16,))
    _cuda_2d(out, "out", _FP8)
    G = w.shape[0]
    ffn = w.shape[2] if b_is_kn else w.shape[1]
    _require(dy.dim() == 2 and w.dim() == 3 and dy.shape[1] == (w.shape[1] if b_is_kn else w.shape[2]),
             "fp8_gmm_dswiglu: contraction dimensions differ")
    _require(len(group_sizes) == G, "fp8_gmm_dswiglu: one group size per expert is required")
    _require(tuple(pre_act.shape) == (dy.shape[0], 2 * ffn) and tuple(out.shape) == (dy.shape[0], 2 * ffn),
             "fp8_gmm_dswiglu: pre_act and out must be (rows, 2 * ffn)")
    sa, sb = _strided(dy_scale_invs, G), _strided(w_scale_invs, G)
    _gemm(dy, w, None, group_sizes, G, sa, sb, ACT_DSWIGLU, out, _strided(out_scales, G),
          _strided(out_amaxes, G, writable=True), b_layout=1 if b_is_kn else 0, aux_in=pre_act)
    return out


_workspaces = {}


def _workspace(device, nbytes):
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(nbytes, 1 << 16), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def grouped_wgrad(a_t, b_t, t_offsets, n, k, a_scale_invs, b_scale_invs, c=None):
    """All weight gradients in one launch: ``c[g] (n, k) = (A_t,g * sa[g]) (B_t,g * sb[g])^T``.

    a_t / b_t are the padded-transposed FP8 buffers produced by the cast kernels (group g is an
    (n x L_g) resp. (k x L_g) row-major block starting at byte t_offsets[g] * n resp. * k), t_offsets
    the host prefix sums of the (16-row padded) group sizes.  Replaces the reference's per-group loop
    (fp8_gmm/grouped_linear.py:165-182).  Empty groups produce zeros.
    """
    G = len(t_offsets) - 1
    _require(a_t.is_cuda and a_t.dtype in _FP8 and b_t.is_cuda and b_t.dtype in _FP8, "grouped_wgrad: FP8 CUDA operands")
    if c is None:
        c = torch.empty(G, n, k, dtype=torch.bfloat16, device=a_t.device)
    _require(tuple(c.shape) == (G, n, k) and c.dtype == torch.bfloat16 and c.is_contiguous(), "grouped_wgrad: bad output")
    args = WgradArgs()
    args.a_t, args.b_t, args.c = a_t.data_ptr(), b_t.data_ptr(), c.data_ptr()
    to, keep = _i64_array(t_offsets)
    args.t_offsets = to
    args.num_groups, args.n, args.k = G, n, k
    args.a_format, args.b_format = _fp8_code(a_t.dtype), _fp8_code(b_t.dtype)
    sa, sb = _strided(a_scale_invs, G), _strided(b_scale_invs, G)
    args.a_scale_inv, args.a_scale_inv_stride = sa.ptr, sa.stride
    args.b_scale_inv, args.b_scale_inv_stride = sb.ptr, sb.stride
    nbytes = lib.fp8gmm_wgrad_workspace_bytes(G)
    ws = _workspace(a_t.device, nbytes)
    args.workspace, args.workspace_bytes = ws.data_ptr(), ws.numel()
    with _Timed(2.0 * a_t.numel() * k):  # a_t holds (padded rows) x n elements
        check(lib.fp8gmm_grouped_wgrad(ctypes.byref(args), _stream()), "grouped_wgrad")
    del keep
    return c


def grouped_wgrad_rowmajor(dy, x, row_offsets, a_scale_invs, b_scale_invs, c=None):
    """All weight gradients in one launch from the row-major FP8 activations, no transposed copies:
    ``c[g] (n, k) = (dy[rows of g] * sa[g])^T (x[rows of g] * sb[g])`` with dy (sum m, n), x (sum m, k) and
    ``row_offsets`` the host prefix sums of the group sizes (any sizes; empty groups give zeros).  Same result as
    ``grouped_wgrad`` on the padded transposes of the same rows (see fp8gmm_grouped_wgrad_rowmajor)."""
    G = len(row_offsets) - 1
    _cuda_2d(dy, "dy", _FP8)
    _cuda_2d(x, "x", _FP8)
    _require(dy.dim() == 2 and x.dim() == 2 and dy.shape[0] == x.shape[0], "grouped_wgrad_rowmajor: row counts differ")
    n, k = dy.shape[1], x.shape[1]
    if c is None:
        c = torch.empty(G, n, k, dtype=torch.bfloat16, device=dy.device)
    _require(tuple(c.shape) == (G, n, k) and c.dtype == torch.bfloat16 and c.is_contiguous(), "grouped_wgrad_rowmajor: bad output")
    args = WgradArgs()
    args.a_t, args.b_t, args.c = dy.data_ptr(), x.data_ptr(), c.data_ptr()
    to, keep = _i64_array(row_offsets)
    args.t_offsets = to
    args.num_groups, args.n, args.k = G, n, k
    args.a_format, args.b_format = _fp8_code(dy.dtype), _fp8_code(x.dtype)
    sa, sb = _strided(a_scale_invs, G), _strided(b_scale_invs, G)
    args.a_scale_inv, args.a_scale_inv_stride = sa.ptr, sa.stride
    args.b_scale_inv, args.b_scale_inv_stride = sb.ptr, sb.stride
    ws = _workspace(dy.device, lib.fp8gmm_wgrad_workspace_bytes(G))
    args.workspace, args.workspace_bytes = ws.data_ptr(), ws.numel()
    with _Timed(2.0 * dy.shape[0] * n * k):
        check(lib.fp8gmm_grouped_wgrad_rowmajor(ctypes.byref(args), _stream()), "grouped_wgrad_rowmajor")
    del keep
    return c


def delayed_scaling_update(amax_history, scale, scale_inv, fp8_max, margin=0, algo="max"):
    """Fused recipe update for one meta set (see fp8gmm_delayed_scaling_update in the header)."""
    _require(amax_history.is_cuda and amax_history.dtype == torch.float32 and amax_history.is_contiguous(),
             "amax_history must be a contiguous CUDA float32 tensor")
    length, n = amax_history.shape
    check(lib.fp8gmm_delayed_scaling_update(amax_history.data_ptr(), scale.data_ptr(), scale_inv.data_ptr(), length, n,
                                            float(fp8_max), float(margin), 0 if algo == "max" else 1, _stream()),
          "delayed_scaling_update")


def device_status():
    """Synchronise the current stream and raise if a kernel reported a bounded wait that ran out."""
    check(lib.fp8gmm_device_status(_stream()), "device_status")


class StatusWatch:
    """Non-blocking view of the device status word for training loops: ``record()`` enqueues a copy of the word
    into page-locked host memory on the current stream, ``check()`` raises if a copy that has already landed shows
    that a bounded wait ran out (the outputs of that launch, and everything computed from them, are undefined)."""

    def __init__(self):
        self.host = torch.zeros(1, dtype=torch.int32).pin_memory()

    def record(self):
        check(lib.fp8gmm_device_status_async(self.host.data_ptr(), _stream()), "device_status_async")

    def check(self):
        code = int(self.host[0])
        if code != 0:
            raise RuntimeError(
                f"fp8_gmm_b200: a kernel gave up on a bounded wait in an earlier step (status 0x{code:x}: a peer was "
                "late or a copy never arrived); results since then are undefined")
