"""GroupedLinear: one FP8 linear layer per group (expert) over row-sorted tokens.

Same surface as reference fp8_gmm/grouped_linear.py (class names, constructor and forward arguments,
saved-tensor layout, meta slots), re-implemented on this package's kernels:

* casts use the grouped C-ABI forms (one base pointer + host prefix sums) instead of Python lists of
  per-group views, so host time does not grow with the number of groups;
* the forward / dgrad GEMM is one launch with the de-scale fused (the reference's CUTLASS path needs a
  second pass, fp8_gmm/backend.py:78-82);
* the weight gradient is one grouped launch (the reference loops over groups, :165-182) that reads the row-major FP8
  activations directly (MN-major tensor-core operands), so the padded transposes the reference builds for it
  (:32-52,:133-149) are not made; FP8GMM_WGRAD=transposed restores that dataflow;
* ``is_first_microbatch`` works (the reference forces None): True casts the weights and keeps the FP8 copies, False
  reuses them and leaves the scales alone, so gradient accumulation pays the weight cast once per optimizer step;
* groups with zero rows are accepted (the reference asserts, :205): they produce no output rows and a
  zero weight gradient.
"""
import math

import torch

from . import backend
from .recipe import Fp8GmmBaseModule, get_fp8_te_dtype
from .utils import Fp8MetaWrapper, Fp8TensorType, MetaTensorType, cumsum_group_sizes, to_torch_dtype

_T, _M = Fp8TensorType, MetaTensorType


class _GroupedLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, weight, group_sizes, fp8_meta, is_grad_enabled, cutlass, weight_cache=None, reuse_weights=False):
        need_wgrad = is_grad_enabled and weight.requires_grad
        need_dgrad = is_grad_enabled and input.requires_grad
        need_t = need_wgrad and not backend.WGRAD_ROWMAJOR   # padded transposes only for the reference's wgrad dataflow
        num_groups, padded, cumsums, padded_cumsums = cumsum_group_sizes(group_sizes.tolist(), need_padding=need_t)
        offs = padded_cumsums if padded else cumsums
        metas = Fp8MetaWrapper(num_groups, fp8_meta)
        dtype = get_fp8_te_dtype(fp8_meta["recipe"], fprop_tensor=True)
        torch_dtype = to_torch_dtype(dtype)
        n, k = weight.shape[1], weight.shape[2]
        assert input.dim() == 2 and input.shape == (cumsums[-1], k), "input must be (sum(group_sizes), in_features)"
        input = input.contiguous()

        input_fp8 = torch.empty(input.shape, dtype=torch_dtype, device=input.device)
        input_t_fp8 = torch.empty(offs[-1], k, dtype=torch_dtype, device=input.device) if need_t else None
        backend.grouped_cast_transpose(
            input, cumsums, input_fp8, input_t_fp8, offs,
            metas.get_meta_strided(_T.kInputGroup1, _M.kScale), metas.get_meta_strided(_T.kInputGroup1, _M.kAmax))
        need_wt = need_dgrad and not backend.DGRAD_KN   # weight transposes only for the reference's dgrad dataflow
        weight_fp8, weight_t_fp8 = cast_weight_cached(
            weight, torch_dtype, need_wt, metas.get_meta_strided(_T.kWeightGroup1, _M.kScale),
            metas.get_meta_strided(_T.kWeightGroup1, _M.kAmax), weight_cache, "weight", reuse_weights)
        out = backend.fp8_gmm(
            input_fp8, weight_fp8, group_sizes,
            metas.get_meta_strided(_T.kInputGroup1, _M.kScaleInv), metas.get_meta_strided(_T.kWeightGroup1, _M.kScaleInv),
            backward=False, cutlass=cutlass)
        if is_grad_enabled:
            ctx.save_for_backward(input_t_fp8 if need_t else (input_fp8 if need_wgrad else None),
                                  weight_t_fp8 if need_wt else (weight_fp8 if need_dgrad else None), group_sizes)
            ctx.need_t, ctx.need_wt = need_t, need_wt
            ctx.num_groups = num_groups
            metas.set_forward_scale_inv_cloned()
            ctx.fp8_meta_wrapper = metas
            ctx.cumsums, ctx.offs = cumsums, offs
            ctx.fp8_meta = fp8_meta
            ctx.weight_shape = weight.shape
            ctx.input_requires_grad = input.requires_grad
            ctx.weight_requires_grad = weight.requires_grad
            ctx.cutlass = cutlass
        return out

    @staticmethod
    def backward(ctx, grad_out):
        input_t_fp8, weight_t_fp8, group_sizes = ctx.saved_tensors
        metas, fp8_meta, cumsums, offs = ctx.fp8_meta_wrapper, ctx.fp8_meta, ctx.cumsums, ctx.offs
        fp8_meta["prepare_backward"]()
        g_dtype = to_torch_dtype(get_fp8_te_dtype(fp8_meta["recipe"], fprop_tensor=False))
        grad_out = grad_out.contiguous()
        _, n, k = ctx.weight_shape
        grad_out_fp8 = torch.empty(grad_out.shape, dtype=g_dtype, device=grad_out.device)
        grad_out_t_fp8 = (torch.empty(offs[-1], n, dtype=g_dtype, device=grad_out.device)
                          if ctx.weight_requires_grad and ctx.need_t else None)
        backend.grouped_cast_transpose(
            grad_out, cumsums, grad_out_fp8, grad_out_t_fp8, offs,
            metas.get_meta_strided(_T.kGradOutputGroup1, _M.kScale), metas.get_meta_strided(_T.kGradOutputGroup1, _M.kAmax))
        grad_input = None
        if ctx.input_requires_grad:
            grad_input = backend.fp8_gmm(
                grad_out_fp8, weight_t_fp8, group_sizes,
                metas.get_meta_strided(_T.kGradOutputGroup1, _M.kScaleInv),
                metas.get_meta_strided(_T.kForwardWeightGroup1, _M.kScaleInv),
                backward=True, cutlass=ctx.cutlass, b_is_kn=not ctx.need_wt)
        grad_weight = None
        if ctx.weight_requires_grad and ctx.need_t:
            grad_weight = backend.grouped_wgrad(
                grad_out_t_fp8, input_t_fp8, offs, n, k,
                metas.get_meta_strided(_T.kGradOutputGroup1, _M.kScaleInv),
                metas.get_meta_strided(_T.kForwardInputGroup1, _M.kScaleInv))
        elif ctx.weight_requires_grad:
            # `input_t_fp8` holds the row-major FP8 input here: the GEMM reads both operands as they lie
            grad_weight = backend.grouped_wgrad_rowmajor(
                grad_out_fp8, input_t_fp8, cumsums,
                metas.get_meta_strided(_T.kGradOutputGroup1, _M.kScaleInv),
                metas.get_meta_strided(_T.kForwardInputGroup1, _M.kScaleInv))
        return grad_input, grad_weight, None, None, None, None, None, None


def cast_weight_cached(weight, fp8_dtype, with_transpose, scale, amax, cache, key, reuse):
    """(G, N, K) bf16 weights -> FP8 copy and, with ``with_transpose``, the per-expert transposes (G, K, N).

    ``cache`` (a dict owned by the module, or None) keeps the FP8 weights between micro-batches: with ``reuse`` the
    cast is skipped when the cached copy fits (same dtype, a transpose present if one is needed).  This is the
    ``is_first_microbatch`` protocol of Transformer Engine modules, which the reference switches off
    (reference fp8_gmm/grouped_linear.py:200-202): weights only change at the optimizer step, so their cast and
    transpose need not be repeated for every micro-batch of a gradient-accumulation step."""
    if cache is not None and reuse and key in cache:
        w_fp8, w_t = cache[key]
        if w_fp8.dtype == fp8_dtype and w_fp8.shape == weight.shape and (w_t is not None or not with_transpose):
            return w_fp8, (w_t if with_transpose else None)
    g, n, k = weight.shape
    w_fp8 = torch.empty(weight.shape, dtype=fp8_dtype, device=weight.device)
    w_t = torch.empty(g, k, n, dtype=fp8_dtype, device=weight.device) if with_transpose else None
    offs = [i * n for i in range(g + 1)]
    backend.grouped_cast_transpose(weight.view(g * n, k), offs, w_fp8, w_t, offs, scale, amax)
    if cache is not None:
        cache[key] = (w_fp8, w_t)
    return w_fp8, w_t


class GroupedLinear(Fp8GmmBaseModule):
    """``out[rows of group g] = input[rows of group g] @ weight[g].T`` in FP8 with delayed scaling.

    Arguments as in reference fp8_gmm/grouped_linear.py:186-214.  ``cutlass`` is accepted for drop-in
    compatibility and has no effect (there is one backend).
    """

    def __init__(self, in_features, out_features, num_groups, dtype, device="cuda", cutlass=False):
        super().__init__()
        assert dtype == torch.bfloat16, "only bfloat16 parameters are supported"
        self.in_features = in_features
        self.out_features = out_features
        self.num_groups = num_groups
        self.weight_tensor = torch.nn.Parameter(
            torch.empty(num_groups, out_features, in_features, dtype=dtype, device=device))
        bound = math.sqrt(1.0 / in_features)
        torch.nn.init.uniform_(self.weight_tensor.data, -bound, bound)
        self.cutlass = cutlass
        self._fp8_weights = {}

    def get_fp8_weights_scratchpad(self, is_first_microbatch):
        """[weight_fp8, weight_t_fp8] kept from the first micro-batch, or [None, None] without caching
        (``is_first_microbatch is None``, the only mode of the reference, fp8_gmm/grouped_linear.py:200-202)."""
        if is_first_microbatch is None:
            self._fp8_weights.clear()
        return list(self._fp8_weights.get("weight", (None, None)))

    def forward(self, input, group_sizes, is_first_microbatch=None):
        if not torch.is_tensor(group_sizes):
            group_sizes = torch.tensor(list(group_sizes), dtype=torch.int64)
        with self.prepare_forward(input, is_first_microbatch, self.num_groups):
            if torch.is_grad_enabled():
                fn, args = _GroupedLinear.apply, []
            else:
                fn, args = _GroupedLinear.forward, [None]
            self.get_fp8_weights_scratchpad(is_first_microbatch)
            args += [input, self.weight_tensor, group_sizes, self.fp8_meta, torch.is_grad_enabled(), self.cutlass,
                     None if is_first_microbatch is None else self._fp8_weights, is_first_microbatch is False]
            return fn(*args)
