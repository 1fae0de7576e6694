"""CPU oracle for the FP8 grouped-GEMM hot path -- TEST INFRASTRUCTURE, never a product fallback.

A torch-on-CPU restatement of what the reference computes on the GPU.  Only ``tests/``,
``__graft_entry__.smoke()`` and the CPU-baseline leg of ``bench.py`` may import this module.

Reference sources restated here (paths relative to the reference project):

* quantise ``OType(scale * fp32(x))``            csrc/multi_pointwise.cu:75-80, csrc/multi_pad_fusion.cu:230-237
* amax of the *unscaled* input, max-merged         csrc/multi_pointwise.cu:78,93-96; csrc/utils.cuh:151-185
* padded-transposed layout                         fp8_gmm/utils.py:48-62; fp8_gmm/grouped_linear.py:32-52,133-149;
                                                   csrc/multi_pad_fusion.cu:268-281
* fp8 -> fp8 padded transpose                      csrc/multi_pad_fusion.cu:46-153; fp8_gmm/test.py:58-70
* dGELU (tanh form)                                csrc/multi_pad_fusion.cu:38-44,378; fp8_gmm/test.py:32-34
* in-place de-scale                                csrc/multi_pointwise.cu:138
* grouped GEMM semantics and operand layouts       csrc/fp8_gmm.h:7-11; csrc/fp8_gmm.cu:101-113,137-144;
                                                   fp8_gmm/backend.py:25-54,72-97
* per-group matmul loop ("the CPU path")           fp8_gmm/test.py:209-214
* GELU-aux epilogue semantics                      fp8_gmm/test.py:159-168,215-229; fp8_gmm/grouped_mlp.py:116-131
* dgrad / wgrad operands and scales                fp8_gmm/grouped_linear.py:154-182; fp8_gmm/grouped_mlp.py:226-322
* meta indexing                                    fp8_gmm/utils.py:80-103

Third-party arithmetic that is absent from the reference checkout and therefore *defined* here:
the grouped GEMM's device code (CUTLASS, un-vendored submodule without a pinned commit) and the
delayed-scaling recipe update plus the cuBLASLt GELU-aux epilogue (Transformer Engine, unpinned,
API generation ~1.x).  For those pieces parity is anchored on the reference's call sites and on the
tolerances of its own tests; the recipe update itself is "parity unpinned".

The quantiser is pinned against the CUDA toolkit's host-side ``__nv_fp8_e4m3`` / ``__nv_fp8_e5m2``
constructors (the converter the reference calls) and, on a GPU machine, against the reference's own
kernels compiled for sm_100a; see tests/test_oracle_pins.py and tests/golden/.
"""
import math

import torch

E4M3 = torch.float8_e4m3fn
E5M2 = torch.float8_e5m2
FP8_MAX = {E4M3: 448.0, E5M2: 57344.0}


# --------------------------------------------------------------------------------------------
# quantise / amax / layouts
# --------------------------------------------------------------------------------------------
def quantize(x, scale, dtype):
    """``OType(scale * fp32(x))``: fp32 product, round-to-nearest-even, saturate to +-max finite.

    torch's CPU cast does not saturate (overflow gives NaN / inf), hence the explicit clamp.  NaN
    becomes the byte 0x7F in both formats with the sign dropped (the converter canonicalises NaN
    first), which torch's cast would not do for negative NaNs.
    """
    scale = float(scale) if not torch.is_tensor(scale) else scale.float()
    y = x.float() * scale
    q = y.clamp(-FP8_MAX[dtype], FP8_MAX[dtype]).to(dtype)
    nan = torch.isnan(y)
    if bool(nan.any()):
        q = torch.where(nan, torch.full_like(q.view(torch.uint8), 0x7F), q.view(torch.uint8)).view(dtype)
    return q


def amax_merge(x, prev=0.0):
    """max(prev, max|fp32(x)|); NaNs are ignored like ``fmaxf`` does."""
    if x.numel() == 0:
        return float(prev)
    a = x.float().abs()
    a = torch.where(torch.isnan(a), torch.zeros_like(a), a)
    return max(float(prev), float(a.max()))


def cumsum_group_sizes(group_sizes, need_padding=False):
    """Prefix sums and per-group round-up to 16 rows (fp8_gmm/utils.py:48-62)."""
    cums, pcs, padded = [0], ([0] if need_padding else None), False
    for g in group_sizes:
        g = int(g)
        cums.append(cums[-1] + g)
        if need_padding:
            r = g % 16
            if r:
                padded = True
                g += 16 - r
            pcs.append(pcs[-1] + g)
    return len(group_sizes), padded, cums, pcs


def pad_transpose(q, padded_rows, pad_byte=0):
    """fp8 (m, n) -> fp8 (n, padded_rows) with ``pad_byte`` in rows >= m."""
    m, n = q.shape
    out = torch.full((n, padded_rows), pad_byte, dtype=torch.uint8)
    out[:, :m] = q.view(torch.uint8).t()
    return out.view(q.dtype)


def pad_byte_for_scale(scale, dtype):
    """The cast kernels compute padding as ``OType(scale * 0)``: -0 (0x80) for a negative scale."""
    return int(quantize(torch.zeros(1, dtype=torch.bfloat16), scale, dtype).view(torch.uint8)[0])


def pad_cast_transpose(x, scale, dtype, padded_rows, prev_amax=0.0, pre_act=None, act="gelu"):
    """Cast + padded transpose (+ optional activation-derivative fusion).

    Returns (out (m,n) fp8, out_t (n,padded_rows) fp8, amax).  With ``pre_act`` given the value
    quantised is ``x * dgelu(pre_act)`` (act="gelu") and the amax is taken over that product.
    """
    v = x.float()
    if pre_act is not None:
        assert act == "gelu"
        v = v * dgelu(pre_act.float())
    q = quantize(v, scale, dtype)
    qt = pad_transpose(q, padded_rows, pad_byte_for_scale(scale, dtype))
    return q, qt, amax_merge(v, prev_amax)


def scale_mul(x, s1, s2):
    """In-place de-scale of the reference's CUTLASS path: bf16(fp32(x) * s1 * s2)."""
    return ((x.float() * float(s1)) * float(s2)).to(torch.bfloat16)


# --------------------------------------------------------------------------------------------
# activations
# --------------------------------------------------------------------------------------------
def gelu(x):
    return 0.5 * x * (1.0 + torch.tanh(0.79788456 * x * (1.0 + 0.044715 * x * x)))


def dgelu(x):
    t = torch.tanh(0.79788456 * x * (1.0 + 0.044715 * x * x))
    return 0.5 * x * ((1.0 - t * t) * (0.79788456 + 0.1070322243 * x * x)) + 0.5 * (1.0 + t)


def swiglu(h):
    """h (m, 2F) = [gate | up] -> silu(gate) * up (extension beyond the reference, which has GELU only)."""
    f = h.shape[1] // 2
    g, u = h[:, :f], h[:, f:]
    return g * torch.sigmoid(g) * u


def dswiglu(dy, h):
    """Gradient of ``swiglu`` w.r.t. h: returns (m, 2F) = [dgate | dup]."""
    f = h.shape[1] // 2
    g, u = h[:, :f], h[:, f:]
    s = torch.sigmoid(g)
    dgate = dy * u * (s * (1.0 + g * (1.0 - s)))
    dup = dy * (g * s)
    return torch.cat([dgate, dup], dim=1)


# --------------------------------------------------------------------------------------------
# grouped GEMMs on dequantised operands, fp32 accumulate, single rounding
# --------------------------------------------------------------------------------------------
def grouped_gemm(a, b, group_sizes, a_scale_invs, b_scale_invs, out_fp32=False):
    """C_g = (A_g * sa_g) (B_g * sb_g)^T per group; A (sum m, K) fp8, B (G, N, K) fp8.

    Mirrors the per-group loop of fp8_gmm/test.py:209-214 but on the *quantised* operands, so it is
    the "fp32 accumulate of the same dequantised operands" that GEMM parity is stated against.
    """
    m_total, n = a.shape[0], b.shape[1]
    c = torch.zeros(m_total, n, dtype=torch.float32)
    start = 0
    for g, m in enumerate(int(s) for s in group_sizes):
        if m:
            acc = a[start : start + m].float() @ b[g].float().t()
            c[start : start + m] = acc * (float(a_scale_invs[g]) * float(b_scale_invs[g]))
        start += m
    return c if out_fp32 else c.to(torch.bfloat16)


def grouped_gemm_act(a, b, group_sizes, a_scale_invs, b_scale_invs, c_scales, prev_amaxes, act="gelu"):
    """fc1 with the activation-aux epilogue: returns (pre_act bf16, act fp8 e4m3, amaxes).

    pre_act = bf16(acc * sa * sb); act = e4m3(act_fn(fp32 pre-activation) * c_scale[g]);
    amax[g] = max(prev, max|act_fn(.)|) over the group's rows.
    """
    h32 = grouped_gemm(a, b, group_sizes, a_scale_invs, b_scale_invs, out_fp32=True)
    fn = gelu if act == "gelu" else swiglu
    n_act = h32.shape[1] if act == "gelu" else h32.shape[1] // 2
    act_q = torch.empty(h32.shape[0], n_act, dtype=E4M3)
    amaxes, start = [], 0
    for g, m in enumerate(int(s) for s in group_sizes):
        v = fn(h32[start : start + m])
        act_q[start : start + m] = quantize(v, c_scales[g], E4M3)
        amaxes.append(amax_merge(v, prev_amaxes[g] if prev_amaxes is not None else 0.0))
        start += m
    return h32.to(torch.bfloat16), act_q, amaxes


def grouped_wgrad(dy_t_blocks, x_t_blocks, dy_scale_invs, x_scale_invs):
    """dW_g (N, K) = dY_g^T X_g computed as (N x Mpad_g) (K x Mpad_g)^T on the padded transposes
    (fp8_gmm/grouped_linear.py:165-182).  Empty groups give zeros."""
    outs = []
    for g, (dyt, xt) in enumerate(zip(dy_t_blocks, x_t_blocks)):
        acc = dyt.float() @ xt.float().t() if dyt.shape[1] else torch.zeros(dyt.shape[0], xt.shape[0])
        outs.append((acc * (float(dy_scale_invs[g]) * float(x_scale_invs[g]))).to(torch.bfloat16))
    return torch.stack(outs)


# --------------------------------------------------------------------------------------------
# delayed-scaling recipe (defined here: Transformer Engine is not part of the reference checkout)
# --------------------------------------------------------------------------------------------
def delayed_scaling_update(amax_history, scale, fp8_max, margin=0, algo="max"):
    """amax = max over history (or most recent); scale = fp8_max / amax / 2^margin where amax is
    positive and finite, else unchanged; scale_inv = 1/scale; history rolled by one with row 0 zeroed."""
    amax = amax_history.max(dim=0).values if algo == "max" else amax_history[0].clone()
    # IEEE division (torch's `scalar / tensor` would multiply by a rounded reciprocal instead)
    sf = torch.full_like(amax, fp8_max) / amax / (2.0**margin)
    sf = torch.where(amax > 0.0, sf, scale)
    sf = torch.where(torch.isfinite(amax), sf, scale)
    if amax_history.shape[0] > 1:
        new_hist = torch.roll(amax_history, -1, 0)
    else:
        new_hist = amax_history.clone()
    new_hist[0].zero_()
    return new_hist, sf, 1.0 / sf


# --------------------------------------------------------------------------------------------
# whole-step oracles (what the autograd functions must reproduce)
# --------------------------------------------------------------------------------------------
def _split(x, cums):
    return [x[cums[i] : cums[i + 1]] for i in range(len(cums) - 1)]


def grouped_linear_step(x, w, dy, group_sizes, x_scales, w_scales, dy_scales):
    """One fwd+bwd of GroupedLinear with given per-group scales (fp8_gmm/grouped_linear.py:11-183).

    x (sum m, K) bf16, w (G, N, K) bf16, dy (sum m, N) bf16.  Returns dict with out, grad_input,
    grad_weight (bf16), the FP8 operands, padded transposes and amaxes.
    """
    G, padded, cums, pcs = cumsum_group_sizes(group_sizes, need_padding=True)
    offs = pcs if padded else cums
    r = {}
    x_q, x_t, x_am, w_q, w_t, w_am = [], [], [], [], [], []
    for g in range(G):
        q, qt, am = pad_cast_transpose(x[cums[g] : cums[g + 1]], x_scales[g], E4M3, offs[g + 1] - offs[g])
        x_q.append(q), x_t.append(qt), x_am.append(am)
        q, qt, am = pad_cast_transpose(w[g], w_scales[g], E4M3, w.shape[1])
        w_q.append(q), w_t.append(qt), w_am.append(am)
    x_fp8 = torch.cat(x_q) if x_q else torch.empty(0, x.shape[1], dtype=E4M3)
    w_fp8, w_t_fp8 = torch.stack(w_q), torch.stack(w_t)
    x_si = [1.0 / float(s) for s in x_scales]
    w_si = [1.0 / float(s) for s in w_scales]
    d_si = [1.0 / float(s) for s in dy_scales]
    r["out"] = grouped_gemm(x_fp8, w_fp8, group_sizes, x_si, w_si)
    dy_q, dy_t, dy_am = [], [], []
    for g in range(G):
        q, qt, am = pad_cast_transpose(dy[cums[g] : cums[g + 1]], dy_scales[g], E5M2, offs[g + 1] - offs[g])
        dy_q.append(q), dy_t.append(qt), dy_am.append(am)
    dy_fp8 = torch.cat(dy_q)
    r["grad_input"] = grouped_gemm(dy_fp8, w_t_fp8, group_sizes, d_si, w_si)
    r["grad_weight"] = grouped_wgrad(dy_t, x_t, d_si, x_si)
    r.update(x_fp8=x_fp8, w_fp8=w_fp8, w_t_fp8=w_t_fp8, dy_fp8=dy_fp8, x_t=x_t, dy_t=dy_t,
             x_amax=x_am, w_amax=w_am, dy_amax=dy_am, padded=padded, cums=cums, offs=offs)
    return r


def grouped_mlp_step(x, w1, w2, dy, group_sizes, scales, act="gelu"):
    """One fwd+bwd of GroupedMlp (fp8_gmm/grouped_mlp.py:18-325) with given per-group scales.

    ``scales`` is a dict of per-group lists: x, w1, act, w2 (forward, e4m3) and dy, dpre (backward,
    e5m2).  act="gelu" follows the reference; act="swiglu" is this repository's extension where w1
    is (G, 2F, H) = [gate rows | up rows].
    """
    G, padded, cums, pcs = cumsum_group_sizes(group_sizes, need_padding=True)
    offs = pcs if padded else cums
    inv = {k: [1.0 / float(s) for s in v] for k, v in scales.items()}

    def cast_groups(t, sc, dt):
        qs, ts, ams = [], [], []
        for g in range(G):
            q, qt, am = pad_cast_transpose(t[cums[g] : cums[g + 1]], sc[g], dt, offs[g + 1] - offs[g])
            qs.append(q), ts.append(qt), ams.append(am)
        return torch.cat(qs), ts, ams

    def cast_weights(w, sc):
        qs, ts, ams = [], [], []
        for g in range(G):
            q, qt, am = pad_cast_transpose(w[g], sc[g], E4M3, w.shape[1])
            qs.append(q), ts.append(qt), ams.append(am)
        return torch.stack(qs), torch.stack(ts), ams

    x_fp8, x_t, x_am = cast_groups(x, scales["x"], E4M3)
    w1_fp8, w1_t, w1_am = cast_weights(w1, scales["w1"])
    w2_fp8, w2_t, w2_am = cast_weights(w2, scales["w2"])
    pre, act_fp8, act_am = grouped_gemm_act(x_fp8, w1_fp8, group_sizes, inv["x"], inv["w1"], scales["act"], None, act)
    out = grouped_gemm(act_fp8, w2_fp8, group_sizes, inv["act"], inv["w2"])
    # backward
    dy_fp8, dy_t, dy_am = cast_groups(dy, scales["dy"], E5M2)
    act_t = [pad_transpose(act_fp8[cums[g] : cums[g + 1]], offs[g + 1] - offs[g]) for g in range(G)]
    grad_w2 = grouped_wgrad(dy_t, act_t, inv["dy"], inv["act"])
    dact = grouped_gemm(dy_fp8, w2_t, group_sizes, inv["dy"], inv["w2"])  # bf16 (sum m, F)
    if act == "gelu":
        dpre_val = dact.float() * dgelu(pre.float())
    else:
        dpre_val = dswiglu(dact.float(), pre.float())
    dq, dts, dam = [], [], []
    for g in range(G):
        v = dpre_val[cums[g] : cums[g + 1]]
        q = quantize(v, scales["dpre"][g], E5M2)
        dq.append(q)
        dts.append(pad_transpose(q, offs[g + 1] - offs[g], pad_byte_for_scale(scales["dpre"][g], E5M2)))
        dam.append(amax_merge(v))
    dpre_fp8 = torch.cat(dq)
    grad_input = grouped_gemm(dpre_fp8, w1_t, group_sizes, inv["dpre"], inv["w1"])
    grad_w1 = grouped_wgrad(dts, x_t, inv["dpre"], inv["x"])
    return dict(out=out, pre=pre, act_fp8=act_fp8, grad_input=grad_input, grad_w1=grad_w1, grad_w2=grad_w2,
                dact=dact, dpre_fp8=dpre_fp8, x_fp8=x_fp8, dy_fp8=dy_fp8,
                amax=dict(x=x_am, w1=w1_am, w2=w2_am, act=act_am, dy=dy_am, dpre=dam))


def rel_frobenius(a, b):
    a, b = a.float(), b.float()
    d = (a - b).norm()
    n = b.norm()
    return float(d / n) if n > 0 else float(d)


def current_scale(x, dtype):
    """fp8_max / amax (1.0 for an all-zero or empty tensor): per-tensor current scaling used by the
    CPU-runnable config."""
    a = amax_merge(x)
    return FP8_MAX[dtype] / a if a > 0 and math.isfinite(a) else 1.0


# ------------------------------------------------------------------------------------------------
# Router-side permutation (reference fp8_gmm/example.py:26-32,52,59: megablocks sort / histogram /
# inclusive_cumsum / gather / scatter, restated from their call sites; megablocks itself is absent: parity unpinned)
# ------------------------------------------------------------------------------------------------
def moe_topk(scores, top_k, moe_renorm=False):
    """Router of the reference's example, verbatim in meaning (fp8_gmm/example.py:14-23): fp32 softmax, torch.topk,
    optional renormalisation.  Returns (multiplier, selected_experts)."""
    weights = torch.nn.functional.softmax(scores, dim=1, dtype=torch.float)
    multiplier, selected = torch.topk(weights, top_k)
    if moe_renorm:
        multiplier = multiplier / multiplier.sum(dim=-1, keepdim=True)
    return multiplier, selected


def moe_sort(top_expert, n_experts):
    """Stable sort of the flat expert ids: (indices, bin_ids, bins, tokens_per_expert, inverse)."""
    ids = top_expert.reshape(-1).to(torch.int64)
    bin_ids, indices = torch.sort(ids, stable=True)
    hist = torch.bincount(ids, minlength=n_experts)
    inverse = torch.empty_like(indices)
    inverse[indices] = torch.arange(ids.numel())
    return indices, bin_ids, torch.cumsum(hist, 0), hist, inverse


def moe_gather(x, indices, top_k, weights=None):
    """out[i] = x[indices[i] // top_k] (times weights[indices[i]], product rounded once to bf16)."""
    rows = x[indices // top_k]
    if weights is None:
        return rows.clone()
    return (rows.float() * weights.reshape(-1).float()[indices, None]).to(x.dtype)


def moe_scatter(x, inverse, top_k, weights=None):
    """out[t] = sum_k w[t, k] * x[inverse[t * top_k + k]]: fp32 fused multiply-adds with k ascending, one rounding."""
    tokens = inverse.numel() // top_k
    acc = torch.zeros(tokens, x.shape[1], dtype=torch.float64)
    w = torch.ones(tokens * top_k) if weights is None else weights.reshape(-1).float()
    for k in range(top_k):
        p = torch.arange(tokens) * top_k + k
        # a float64 multiply-add rounded to float32 equals the fused fp32 multiply-add of the kernel
        acc = (w[p, None].double() * x[inverse[p]].double() + acc).float().double()
    return acc.float().to(x.dtype)
