"""GroupedMlp: per-group two-layer MLP (fc1 -> activation -> fc2) in FP8 over row-sorted tokens.

Surface of reference fp8_gmm/grouped_mlp.py (GroupedMlp(in_features, out_features, num_groups, dtype,
device).forward(input, group_sizes, has_tp, tp_group, is_first_microbatch)) plus
``activation={"gelu","swiglu"}``.  Dataflow follows the reference's autograd function (:18-325):
fc1 with the activation fused in the GEMM epilogue (pre-activation bf16 + e4m3 activation + amax), fc2,
and in backward fc2 wgrad / fc2 dgrad / fused d-activation cast / fc1 dgrad (optionally all-reduced
over a tensor-parallel group, overlapped with fc1 wgrad) / fc1 wgrad.  Every per-group cuBLASLt loop
of the reference is one grouped launch here.  ``GroupedMLP`` is an alias.
"""
import math

import torch

from . import backend, tp
from .grouped_linear import cast_weight_cached
from .recipe import Fp8GmmBaseModule, get_fp8_te_dtype
from .utils import Fp8MetaWrapper, Fp8TensorType, MetaTensorType, cumsum_group_sizes, to_torch_dtype

_T, _M = Fp8TensorType, MetaTensorType
# chunks of experts the fc1 data-gradient GEMM is cut into when its result is summed over a tensor-parallel group
TP_CHUNKS = 4


class _GroupedMlp(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, fc1_weight, fc2_weight, group_sizes, fp8_meta, is_grad_enabled, has_tp, tp_group, activation,
                perm=None, weight_cache=None, reuse_weights=False):
        input_requires_grad = input.requires_grad
        weight_requires_grad = fc1_weight.requires_grad
        need_wgrad = is_grad_enabled and weight_requires_grad
        need_dgrad = is_grad_enabled and input_requires_grad
        need_t = need_wgrad and not backend.WGRAD_ROWMAJOR   # padded transposes only for the reference's wgrad dataflow
        num_groups, padded, cumsums, padded_cumsums = cumsum_group_sizes(group_sizes.tolist(), need_padding=need_t)
        offs = padded_cumsums if padded else cumsums
        metas = Fp8MetaWrapper(num_groups, fp8_meta)
        torch_dtype = to_torch_dtype(get_fp8_te_dtype(fp8_meta["recipe"], fprop_tensor=True))
        hidden = input.shape[1]
        fc1_out = fc1_weight.shape[1]                       # F (gelu) or 2F (swiglu)
        ffn = fc1_out // 2 if activation == "swiglu" else fc1_out
        assert fc2_weight.shape[2] == ffn and fc2_weight.shape[1] == hidden
        assert input.dim() == 2 and input.shape[0] == cumsums[-1]
        input = input.contiguous()

        input_fp8 = torch.empty(input.shape, dtype=torch_dtype, device=input.device)
        input_t_fp8 = torch.empty(offs[-1], hidden, dtype=torch_dtype, device=input.device) if need_t else None
        x_scale, x_amax = metas.get_meta_strided(_T.kInputGroup1, _M.kScale), metas.get_meta_strided(_T.kInputGroup1, _M.kAmax)
        if perm is None:
            backend.grouped_cast_transpose(input, cumsums, input_fp8, input_t_fp8, offs, x_scale, x_amax)
        else:
            # rows arrive in an external (source-major) order: the cast itself puts them expert-major
            backend.blocked_cast(input, input_fp8, perm, x_scale, x_amax, num_groups)
            if need_t:
                backend.grouped_cast_transpose(input_fp8, cumsums, None, input_t_fp8, offs, None, None)
        kn = backend.DGRAD_KN   # dgrad multiplies by the forward FP8 weights as they are: no weight transposes
        fc1_w_fp8, fc1_w_t = cast_weight_cached(
            fc1_weight, torch_dtype, need_dgrad and not kn,
            metas.get_meta_strided(_T.kWeightGroup1, _M.kScale), metas.get_meta_strided(_T.kWeightGroup1, _M.kAmax),
            weight_cache, "fc1", reuse_weights)
        # d(activation) feeds the fc1 weight gradient too, so fc2's transpose is needed whenever anything trains
        fc2_w_fp8, fc2_w_t = cast_weight_cached(
            fc2_weight, torch_dtype, (need_dgrad or need_wgrad) and not kn,
            metas.get_meta_strided(_T.kWeightGroup2, _M.kScale), metas.get_meta_strided(_T.kWeightGroup2, _M.kAmax),
            weight_cache, "fc2", reuse_weights)

        pre_act = torch.empty(input.shape[0], fc1_out, dtype=torch.bfloat16, device=input.device)
        act_fp8 = torch.empty(input.shape[0], ffn, dtype=torch_dtype, device=input.device)
        backend.fp8_gmm(
            input_fp8, fc1_w_fp8, group_sizes,
            metas.get_meta_strided(_T.kInputGroup1, _M.kScaleInv), metas.get_meta_strided(_T.kWeightGroup1, _M.kScaleInv),
            c=act_fp8, pre_gelu_out=pre_act,
            c_scales=metas.get_meta_strided(_T.kInputGroup2, _M.kScale),
            c_amaxes=metas.get_meta_strided(_T.kInputGroup2, _M.kAmax),
            backward=False, activation=activation)
        out = backend.fp8_gmm(
            act_fp8, fc2_w_fp8, group_sizes,
            metas.get_meta_strided(_T.kInputGroup2, _M.kScaleInv), metas.get_meta_strided(_T.kWeightGroup2, _M.kScaleInv),
            backward=False, c_row_map=None if perm is None else perm.row_map)
        if is_grad_enabled:
            ctx.save_for_backward(input_t_fp8 if need_t else (input_fp8 if need_wgrad else None),
                                  (fc1_w_fp8 if need_dgrad else None) if kn else fc1_w_t, fc2_w_fp8 if kn else fc2_w_t, pre_act,
                                  act_fp8 if need_wgrad else None, group_sizes)
            ctx.need_t, ctx.kn = need_t, kn
            ctx.num_groups = num_groups
            metas.set_forward_scale_inv_cloned()
            ctx.fp8_meta_wrapper = metas
            ctx.cumsums, ctx.offs = cumsums, offs
            ctx.fp8_meta = fp8_meta
            ctx.fc1_weight_shape, ctx.fc2_weight_shape = fc1_weight.shape, fc2_weight.shape
            ctx.input_requires_grad, ctx.weight_requires_grad = input_requires_grad, weight_requires_grad
            ctx.has_tp = has_tp
            if has_tp:
                assert tp_group is not None
            ctx.tp_group = tp_group
            ctx.activation = activation
            ctx.perm = perm
        return out

    @staticmethod
    def backward(ctx, grad_out):
        input_t_fp8, fc1_w_t, fc2_w_t, pre_act, act_fp8, group_sizes = ctx.saved_tensors
        metas, fp8_meta, cumsums, offs = ctx.fp8_meta_wrapper, ctx.fp8_meta, ctx.cumsums, ctx.offs
        fp8_meta["prepare_backward"]()
        g_dtype = to_torch_dtype(get_fp8_te_dtype(fp8_meta["recipe"], fprop_tensor=False))
        grad_out = grad_out.contiguous()
        _, fc1_out, hidden = ctx.fc1_weight_shape
        ffn = ctx.fc2_weight_shape[2]
        dev = grad_out.device
        wgrad = ctx.weight_requires_grad
        need_t = wgrad and ctx.need_t

        perm = ctx.perm
        grad_out_fp8 = torch.empty(grad_out.shape, dtype=g_dtype, device=dev)
        grad_out_t = torch.empty(offs[-1], hidden, dtype=g_dtype, device=dev) if need_t else None
        dy_scale, dy_amax = (metas.get_meta_strided(_T.kGradOutputGroup1, _M.kScale),
                             metas.get_meta_strided(_T.kGradOutputGroup1, _M.kAmax))
        if perm is None:
            backend.grouped_cast_transpose(grad_out, cumsums, grad_out_fp8, grad_out_t, offs, dy_scale, dy_amax)
        else:
            backend.blocked_cast(grad_out, grad_out_fp8, perm, dy_scale, dy_amax, ctx.num_groups)
            if need_t:
                backend.grouped_cast_transpose(grad_out_fp8, cumsums, None, grad_out_t, offs, None, None)
        dy_scale_inv = metas.get_meta_strided(_T.kGradOutputGroup1, _M.kScaleInv)
        grad_fc2_weight = None
        if need_t:
            act_t = torch.empty(offs[-1], ffn, dtype=act_fp8.dtype, device=dev)
            backend.grouped_cast_transpose(act_fp8, cumsums, None, act_t, offs, None, None)
            grad_fc2_weight = backend.grouped_wgrad(
                grad_out_t, act_t, offs, hidden, ffn, dy_scale_inv,
                metas.get_meta_strided(_T.kForwardInputGroup2, _M.kScaleInv))
        elif wgrad:
            grad_fc2_weight = backend.grouped_wgrad_rowmajor(
                grad_out_fp8, act_fp8, cumsums, dy_scale_inv, metas.get_meta_strided(_T.kForwardInputGroup2, _M.kScaleInv))
        grad_pre_fp8 = torch.empty(pre_act.shape, dtype=g_dtype, device=dev)
        grad_pre_t = torch.empty(offs[-1], fc1_out, dtype=g_dtype, device=dev) if need_t else None
        dpre_scale, dpre_amax = (metas.get_meta_strided(_T.kGradOutputGroup2, _M.kScale),
                                 metas.get_meta_strided(_T.kGradOutputGroup2, _M.kAmax))
        if ctx.activation == "swiglu" and not need_t and backend.FUSED_DSWIGLU:
            # fc2 dgrad with the SwiGLU backward, the cast and the amax in its epilogue: d(act) never goes to memory
            backend.fp8_gmm_dswiglu(
                grad_out_fp8, fc2_w_t, group_sizes, dy_scale_inv,
                metas.get_meta_strided(_T.kForwardWeightGroup2, _M.kScaleInv), pre_act, grad_pre_fp8, dpre_scale, dpre_amax,
                b_is_kn=ctx.kn)
        else:
            grad_act = backend.fp8_gmm(
                grad_out_fp8, fc2_w_t, group_sizes, dy_scale_inv,
                metas.get_meta_strided(_T.kForwardWeightGroup2, _M.kScaleInv), backward=True, b_is_kn=ctx.kn)
            # d(activation) fused with the e5m2 cast, the padded transpose and the amax
            backend.grouped_cast_transpose(
                grad_act, cumsums, grad_pre_fp8, grad_pre_t, offs, dpre_scale, dpre_amax, in2=pre_act, activation=ctx.activation)
        dpre_scale_inv = metas.get_meta_strided(_T.kGradOutputGroup2, _M.kScaleInv)
        grad_input, handle, reducer = None, None, None
        if ctx.input_requires_grad and ctx.has_tp and perm is None and tp.use_peer_reduction(ctx.tp_group):
            # Tensor-parallel sum over peer memory, chunk by chunk behind the GEMM that produces the partial rows:
            # each chunk of experts is written into the peer-mapped staging buffer and summed on a side stream while
            # the next chunk and the fc1 weight gradient keep the tensor cores busy (fp8_gmm_b200/tp.py).
            reducer = tp.TpReducer.setup(dev, ctx.tp_group)
            rows = cumsums[-1]
            partial = reducer.begin(rows, hidden)
            grad_input = torch.empty(rows, hidden, dtype=torch.bfloat16, device=dev)
            for j0, j1 in tp.chunk_groups(cumsums, TP_CHUNKS):
                r0, r1 = cumsums[j0], cumsums[j1]
                if r1 > r0:
                    backend.fp8_gmm(
                        grad_pre_fp8[r0:r1], fc1_w_t[j0:j1], group_sizes[j0:j1],
                        metas.get_meta_strided(_T.kGradOutputGroup2, _M.kScaleInv, j0),
                        metas.get_meta_strided(_T.kForwardWeightGroup1, _M.kScaleInv, j0), c=partial[r0:r1], backward=True,
                        b_is_kn=ctx.kn)
                    reducer.reduce_rows(grad_input, r0, r1)
        elif ctx.input_requires_grad:
            grad_input = backend.fp8_gmm(
                grad_pre_fp8, fc1_w_t, group_sizes, dpre_scale_inv,
                metas.get_meta_strided(_T.kForwardWeightGroup1, _M.kScaleInv), backward=True,
                c_row_map=None if perm is None else perm.row_map, b_is_kn=ctx.kn)
            if ctx.has_tp:
                handle = torch.distributed.all_reduce(
                    grad_input, op=torch.distributed.ReduceOp.SUM, group=ctx.tp_group, async_op=True)
        grad_fc1_weight = None
        if need_t:
            grad_fc1_weight = backend.grouped_wgrad(
                grad_pre_t, input_t_fp8, offs, fc1_out, hidden, dpre_scale_inv,
                metas.get_meta_strided(_T.kForwardInputGroup1, _M.kScaleInv))
        elif wgrad:
            # `input_t_fp8` holds the row-major FP8 input here
            grad_fc1_weight = backend.grouped_wgrad_rowmajor(
                grad_pre_fp8, input_t_fp8, cumsums, dpre_scale_inv, metas.get_meta_strided(_T.kForwardInputGroup1, _M.kScaleInv))
        if handle is not None:
            handle.wait()
        if reducer is not None:
            reducer.finish()
        return grad_input, grad_fc1_weight, grad_fc2_weight, None, None, None, None, None, None, None, None, None


class GroupedMlp(Fp8GmmBaseModule):
    """Per-group MLP.  ``fc1_weight`` is (G, out_features, in_features) for GELU (as in the reference) and
    (G, 2*out_features, in_features) = [gate rows | up rows] for SwiGLU; ``fc2_weight`` is
    (G, in_features, out_features)."""

    def __init__(self, in_features, out_features, num_groups, dtype, device="cuda", activation="gelu"):
        super().__init__()
        assert dtype == torch.bfloat16, "only bfloat16 parameters are supported"
        assert activation in ("gelu", "swiglu")
        self.num_groups = num_groups
        self.activation = activation
        fc1_rows = out_features * (2 if activation == "swiglu" else 1)
        self.fc1_weight = torch.nn.Parameter(torch.empty(num_groups, fc1_rows, in_features, dtype=dtype, device=device))
        self.fc2_weight = torch.nn.Parameter(torch.empty(num_groups, in_features, out_features, dtype=dtype, device=device))
        b1, b2 = math.sqrt(1.0 / in_features), math.sqrt(1.0 / out_features)
        torch.nn.init.uniform_(self.fc1_weight.data, -b1, b1)
        torch.nn.init.uniform_(self.fc2_weight.data, -b2, b2)
        self._fp8_weights = {}

    def get_fp8_weights_scratchpad(self, is_first_microbatch):
        """[fc1_fp8, fc1_t_fp8, fc2_fp8, fc2_t_fp8] kept from the first micro-batch, or Nones without caching
        (``is_first_microbatch is None``, the only mode of the reference, fp8_gmm/grouped_mlp.py:343-345)."""
        if is_first_microbatch is None:
            self._fp8_weights.clear()
        return list(self._fp8_weights.get("fc1", (None, None))) + list(self._fp8_weights.get("fc2", (None, None)))

    def forward(self, input, group_sizes, has_tp=False, tp_group=None, is_first_microbatch=None, row_permutation=None):
        """``row_permutation`` (a backend.RowPermutation, optional, not in the reference): rows of ``input`` and of
        the result are in an external block order (e.g. as an all-to-all delivers them) instead of sorted by group;
        the casts and the GEMM epilogues apply the permutation, so no separate gather / scatter pass runs."""
        if not torch.is_tensor(group_sizes):
            group_sizes = torch.tensor(list(group_sizes), dtype=torch.int64)
        with self.prepare_forward(input, is_first_microbatch, self.num_groups * 2):
            if torch.is_grad_enabled():
                fn, args = _GroupedMlp.apply, []
            else:
                fn, args = _GroupedMlp.forward, [None]
            self.get_fp8_weights_scratchpad(is_first_microbatch)
            args += [input, self.fc1_weight, self.fc2_weight, group_sizes, self.fp8_meta, torch.is_grad_enabled(),
                     has_tp, tp_group, self.activation, row_permutation,
                     None if is_first_microbatch is None else self._fp8_weights, is_first_microbatch is False]
            return fn(*args)


GroupedMLP = GroupedMlp
