"""Router-side steps of an MoE block: sort rows by expert, gather them, scatter the results back.

The reference's example takes these from megablocks (``mega_ops.sort / histogram / inclusive_cumsum / gather /
scatter``, reference fp8_gmm/example.py:26-32,52,59); megablocks is not a dependency of this package, so the same
calls are provided here on this package's kernels (fp8_gmm_b200/csrc/routing.cu), with the same argument order:

    multiplier, selected_experts = topk(scores, top_k, moe_renorm)
    indices, bin_ids, bins, tokens_per_expert = indices_and_bins(top_experts, n_experts)
    rows = gather(x, indices, bin_ids, bins, top_k)             # rows sorted by expert: what GroupedMlp consumes
    out = scatter(expert_out, indices, bin_ids, weights, bins, top_k)

``gather`` and ``scatter`` are differentiable (w.r.t. the rows and, for scatter, the router weights), ``topk`` w.r.t.
the logits.
"""
import torch

from ._lib import check, lib
from .backend import _stream


class Routing:
    """Result of the sort: ``indices`` (stable argsort of the flat expert ids), ``bin_ids`` (sorted expert ids),
    ``bins`` (inclusive cumsum of the histogram), ``tokens_per_expert`` and the inverse permutation."""

    __slots__ = ("indices", "bin_ids", "bins", "tokens_per_expert", "inverse")

    def __init__(self, indices, bin_ids, bins, tokens_per_expert, inverse):
        self.indices, self.bin_ids, self.bins = indices, bin_ids, bins
        self.tokens_per_expert, self.inverse = tokens_per_expert, inverse


class _TopK(torch.autograd.Function):
    @staticmethod
    def forward(ctx, scores, top_k, renorm):
        scores = scores.contiguous()
        tokens, n_experts = scores.shape
        dev = scores.device
        probs = torch.empty(tokens, n_experts, dtype=torch.float32, device=dev)
        weights = torch.empty(tokens, top_k, dtype=torch.float32, device=dev)
        experts = torch.empty(tokens, top_k, dtype=torch.int32, device=dev)
        check(lib.fp8gmm_moe_topk(scores.data_ptr(), int(scores.dtype == torch.bfloat16), tokens, n_experts, top_k, int(renorm),
                                  probs.data_ptr(), weights.data_ptr(), experts.data_ptr(), _stream()), "moe_topk")
        picked = experts.long()
        ctx.save_for_backward(probs, picked, weights)
        ctx.renorm, ctx.in_dtype = renorm, scores.dtype
        ctx.mark_non_differentiable(picked)
        return weights, picked

    @staticmethod
    def backward(ctx, grad_w, _):
        # (tokens x experts) is tiny next to the rows: plain torch ops
        probs, picked, weights = ctx.saved_tensors
        grad_w = grad_w.float()
        if ctx.renorm:   # weights = p_sel / sum(p_sel)
            p_sel = probs.gather(1, picked)
            total = p_sel.sum(1, keepdim=True)
            grad_w = (grad_w - (grad_w * weights).sum(1, keepdim=True)) / total
        grad_p = torch.zeros_like(probs).scatter_(1, picked, grad_w)
        grad_logits = probs * (grad_p - (grad_p * probs).sum(1, keepdim=True))
        return grad_logits.to(ctx.in_dtype), None, None


def topk(scores, top_k, moe_renorm=False):
    """Router of the reference's example (fp8_gmm/example.py:14-23) as one kernel: softmax over the experts in fp32,
    the ``top_k`` largest probabilities (descending) and their expert ids, renormalised to sum to one when
    ``moe_renorm``.  ``scores``: (tokens, n_experts) CUDA float32 or bfloat16.  Returns (multiplier fp32
    (tokens, top_k), selected_experts int64 (tokens, top_k)); any top_k up to n_experts (the reference asserts 1 or 2)."""
    assert scores.is_cuda and scores.dim() == 2 and scores.dtype in (torch.float32, torch.bfloat16)
    return _TopK.apply(scores, int(top_k), bool(moe_renorm))


def sort_by_expert(top_expert, n_experts):
    """top_expert: CUDA integer tensor with tokens * top_k expert ids (flattened token-major).  Returns a Routing."""
    ids = top_expert.reshape(-1).to(torch.int32).contiguous()
    assert ids.is_cuda, "routing runs on CUDA tensors only"
    n = ids.numel()
    dev = ids.device
    indices = torch.empty(n, dtype=torch.int32, device=dev)
    bin_ids = torch.empty(n, dtype=torch.int32, device=dev)
    inverse = torch.empty(n, dtype=torch.int32, device=dev)
    bins = torch.empty(n_experts, dtype=torch.int64, device=dev)
    hist = torch.empty(n_experts, dtype=torch.int64, device=dev)
    check(lib.fp8gmm_moe_sort(ids.data_ptr(), n, n_experts, indices.data_ptr(), bin_ids.data_ptr(), inverse.data_ptr(),
                              bins.data_ptr(), hist.data_ptr(), _stream()), "moe_sort")
    # the megablocks-style calls below only pass `indices` on: let it carry its inverse permutation
    indices._fp8gmm_inverse = inverse
    return Routing(indices, bin_ids, bins, hist, inverse)


def indices_and_bins(top_expert, n_experts, sort_end_bit=None):
    """Same return order as the reference example's helper (fp8_gmm/example.py:26-32): indices, bin_ids, bins,
    tokens_per_expert.  ``sort_end_bit`` is accepted and ignored (the counting sort needs no bit count)."""
    r = sort_by_expert(top_expert, n_experts)
    return r.indices, r.bin_ids, r.bins, r.tokens_per_expert


def _inverse(indices):
    inv = getattr(indices, "_fp8gmm_inverse", None)
    if inv is None:  # an `indices` tensor that did not come from sort_by_expert: invert it here
        inv = torch.empty_like(indices)
        inv[indices.long()] = torch.arange(indices.numel(), dtype=indices.dtype, device=indices.device)
    return inv


def _gather_raw(x, indices, weights, top_k):
    x = x.contiguous()
    out = torch.empty(indices.numel(), x.shape[1], dtype=x.dtype, device=x.device)
    check(lib.fp8gmm_moe_gather(x.data_ptr(), indices.data_ptr(), None if weights is None else weights.data_ptr(), top_k,
                                indices.numel(), x.shape[1], out.data_ptr(), _stream()), "moe_gather")
    return out


def _scatter_raw(x, inverse, weights, top_k):
    x = x.contiguous()
    tokens = inverse.numel() // top_k
    out = torch.empty(tokens, x.shape[1], dtype=x.dtype, device=x.device)
    check(lib.fp8gmm_moe_scatter(x.data_ptr(), inverse.data_ptr(), None if weights is None else weights.data_ptr(), top_k,
                                 tokens, x.shape[1], out.data_ptr(), _stream()), "moe_scatter")
    return out


class _Gather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, indices, inverse, top_k):
        ctx.save_for_backward(inverse)
        ctx.top_k = top_k
        return _gather_raw(x, indices, None, top_k)

    @staticmethod
    def backward(ctx, grad):
        (inverse,) = ctx.saved_tensors
        return _scatter_raw(grad, inverse, None, ctx.top_k), None, None, None


class _Scatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, indices, inverse, weights, top_k):
        w = None if weights is None else weights.reshape(-1).float().contiguous()
        ctx.save_for_backward(x, indices, inverse, w)
        ctx.top_k, ctx.w_dtype = top_k, None if weights is None else weights.dtype
        ctx.w_shape = None if weights is None else weights.shape
        return _scatter_raw(x, inverse, w, top_k)

    @staticmethod
    def backward(ctx, grad):
        x, indices, inverse, w = ctx.saved_tensors
        grad = grad.contiguous()
        grad_x = _gather_raw(grad, indices, w, ctx.top_k) if ctx.needs_input_grad[0] else None
        grad_w = None
        if w is not None and ctx.needs_input_grad[3]:
            grad_w = torch.empty(inverse.numel(), dtype=torch.float32, device=grad.device)
            check(lib.fp8gmm_moe_rowdot(grad.data_ptr(), x.contiguous().data_ptr(), inverse.data_ptr(), ctx.top_k,
                                        inverse.numel(), x.shape[1], grad_w.data_ptr(), _stream()), "moe_rowdot")
            grad_w = grad_w.to(ctx.w_dtype).reshape(ctx.w_shape)
        return grad_x, None, None, grad_w, None


def gather(x, indices, bin_ids, bins, top_k):
    """(tokens, hidden) bf16 -> (tokens * top_k, hidden) rows sorted by expert: out[i] = x[indices[i] // top_k]."""
    assert x.dtype == torch.bfloat16 and x.dim() == 2 and x.is_cuda
    return _Gather.apply(x, indices, _inverse(indices), top_k)


def scatter(x, indices, bin_ids, weights, bins, top_k):
    """(tokens * top_k, hidden) expert-sorted rows -> (tokens, hidden): out[t] = sum_k weights[t*top_k+k] * x[row of
    (t, k)] (fp32 accumulation, one rounding).  ``weights``: tokens * top_k router weights (any float dtype) or None."""
    assert x.dtype == torch.bfloat16 and x.dim() == 2 and x.is_cuda
    return _Scatter.apply(x, indices, _inverse(indices), weights, top_k)
