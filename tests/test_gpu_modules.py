"""GPU: GroupedLinear / GroupedMlp forward + backward against the whole-step CPU oracle, the
delayed-scaling hooks across steps, and checkpoint round trips.

The reference has no module-level tests (fp8_gmm/test.py covers backend ops only), so these are
written from the autograd functions' dataflow (fp8_gmm/grouped_linear.py:11-183,
fp8_gmm/grouped_mlp.py:18-325) restated in oracle/oracle.py.
"""
import copy

import pytest
import torch

from oracle import oracle as O
from tests.helpers import randn_bf16, routed_group_sizes, u8

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _first_step_scales(G, n_fwd=3, n_bwd=2):
    # the first step of delayed scaling runs with scale = 1 everywhere
    return [1.0] * G


@pytest.mark.parametrize("sizes,k,n", [([128, 96, 160, 128], 512, 1024), ([5, 0, 33, 130], 64, 48)])
def test_grouped_linear_first_step_matches_oracle(cuda, wgrad_dataflow, sizes, k, n):
    import fp8_gmm_b200 as fg

    G, m = len(sizes), sum(sizes)
    x = randn_bf16((m, k), 0)
    w = randn_bf16((G, n, k), 1, std=0.02)
    dy = randn_bf16((m, n), 2)
    layer = fg.GroupedLinear(k, n, G, torch.bfloat16, device=cuda)
    with torch.no_grad():
        layer.weight_tensor.copy_(w)
    xin = x.to(cuda).requires_grad_(True)
    with fg.fp8_autocast(enabled=True, fp8_recipe=fg.DelayedScaling(amax_history_len=4)):
        out = layer(xin, torch.tensor(sizes))
    out.backward(dy.to(cuda))
    fg.backend.device_status()
    ones = _first_step_scales(G)
    ref = O.grouped_linear_step(x, w, dy, sizes, ones, ones, ones)
    assert O.rel_frobenius(out.detach().cpu(), ref["out"]) <= 4e-3
    assert O.rel_frobenius(xin.grad.cpu(), ref["grad_input"]) <= 4e-3
    assert O.rel_frobenius(layer.weight_tensor.grad.cpu(), ref["grad_weight"]) <= 4e-3
    for g, s in enumerate(sizes):
        if s == 0:
            assert (layer.weight_tensor.grad[g] == 0).all()
    # amaxes recorded in the history's newest row, at the reference's slots (fp8_gmm/utils.py:98-103)
    fwd = layer.fp8_meta["scaling_fwd"].amax_history[0].cpu()
    bwd = layer.fp8_meta["scaling_bwd"].amax_history[0].cpu()
    for g in range(G):
        assert float(fwd[3 * g]) == ref["x_amax"][g]
        assert float(fwd[3 * g + 1]) == ref["w_amax"][g]
        assert float(bwd[2 * g]) == ref["dy_amax"][g]


def test_grouped_linear_delayed_scaling_second_step(cuda):
    """Step 2 must quantise with scale = fp8_max / amax(step 1) and de-scale consistently."""
    import fp8_gmm_b200 as fg

    sizes, k, n = [40, 24], 64, 32
    G, m = 2, 64
    w = randn_bf16((G, n, k), 1, std=0.02)
    layer = fg.GroupedLinear(k, n, G, torch.bfloat16, device=cuda)
    with torch.no_grad():
        layer.weight_tensor.copy_(w)
    rec = fg.DelayedScaling(amax_history_len=16, margin=0)
    xs = [randn_bf16((m, k), 10 + i) for i in range(2)]
    dys = [randn_bf16((m, n), 20 + i) for i in range(2)]
    refs = []
    for step in range(2):
        xin = xs[step].to(cuda).requires_grad_(True)
        layer.weight_tensor.grad = None
        with fg.fp8_autocast(enabled=True, fp8_recipe=rec):
            out = layer(xin, torch.tensor(sizes))
        out.backward(dys[step].to(cuda))
        if step == 0:
            sx = sw = sd = [1.0] * G
        else:
            prev = refs[0]
            sx = [448.0 / a for a in prev["x_amax"]]
            sw = [448.0 / a for a in prev["w_amax"]]
            sd = [57344.0 / a for a in prev["dy_amax"]]
        ref = O.grouped_linear_step(xs[step], w, dys[step], sizes, [torch.tensor(s) for s in sx],
                                    [torch.tensor(s) for s in sw], [torch.tensor(s) for s in sd])
        refs.append(ref)
        assert O.rel_frobenius(out.detach().cpu(), ref["out"]) <= 4e-3
        assert O.rel_frobenius(xin.grad.cpu(), ref["grad_input"]) <= 4e-3
        assert O.rel_frobenius(layer.weight_tensor.grad.cpu(), ref["grad_weight"]) <= 4e-3
    assert torch.allclose(layer.fp8_meta["scaling_fwd"].scale[0::3].cpu(), torch.tensor([448.0 / a for a in refs[0]["x_amax"]]))
    assert layer.fp8_meta["scaling_fwd"].amax_history.shape == (16, 3 * G)


def _mlp_oracle_scales(G):
    one = [1.0] * G
    return dict(x=one, w1=one, act=one, w2=one, dy=one, dpre=one)


@pytest.mark.parametrize("act", ["gelu", "swiglu"])
@pytest.mark.parametrize("sizes,h,f", [([128, 96, 160, 128], 256, 512), ([5, 0, 33, 130], 64, 96)])
def test_grouped_mlp_first_step_matches_oracle(cuda, wgrad_dataflow, act, sizes, h, f):
    import fp8_gmm_b200 as fg

    G, m = len(sizes), sum(sizes)
    x = randn_bf16((m, h), 0)
    w1 = randn_bf16((G, f * (2 if act == "swiglu" else 1), h), 1, std=0.05)
    w2 = randn_bf16((G, h, f), 2, std=0.05)
    dy = randn_bf16((m, h), 3)
    mlp = fg.GroupedMlp(h, f, G, torch.bfloat16, device=cuda, activation=act)
    with torch.no_grad():
        mlp.fc1_weight.copy_(w1)
        mlp.fc2_weight.copy_(w2)
    xin = x.to(cuda).requires_grad_(True)
    with fg.fp8_autocast(enabled=True, fp8_recipe=fg.DelayedScaling(amax_history_len=2)):
        out = mlp(xin, torch.tensor(sizes))
    out.backward(dy.to(cuda))
    fg.backend.device_status()
    ref = O.grouped_mlp_step(x, w1, w2, dy, sizes, _mlp_oracle_scales(G), act=act)
    # fp8 re-quantisation of intermediates amplifies last-bit differences of the fused activations:
    # every tensor is still held to the 1e-2 bar of the GEMM contract
    assert O.rel_frobenius(out.detach().cpu(), ref["out"]) <= TOL
    assert O.rel_frobenius(xin.grad.cpu(), ref["grad_input"]) <= TOL
    assert O.rel_frobenius(mlp.fc1_weight.grad.cpu(), ref["grad_w1"]) <= TOL
    assert O.rel_frobenius(mlp.fc2_weight.grad.cpu(), ref["grad_w2"]) <= TOL
    fwd = mlp.fp8_meta["scaling_fwd"].amax_history[0].cpu()
    bwd = mlp.fp8_meta["scaling_bwd"].amax_history[0].cpu()
    for g in range(G):
        assert float(fwd[3 * g]) == ref["amax"]["x"][g]
        assert float(fwd[3 * g + 1]) == ref["amax"]["w1"][g]
        assert float(fwd[3 * (G + g) + 1]) == ref["amax"]["w2"][g]
        assert abs(float(fwd[3 * (G + g)]) - ref["amax"]["act"][g]) <= 1e-2 * max(ref["amax"]["act"][g], 1e-6)
        assert float(bwd[2 * g]) == ref["amax"]["dy"][g]
        assert abs(float(bwd[2 * (G + g)]) - ref["amax"]["dpre"][g]) <= 2e-2 * max(ref["amax"]["dpre"][g], 1e-6)


def test_no_grad_forward_and_frozen_weights(cuda):
    import fp8_gmm_b200 as fg

    sizes, h, f = [48, 16], 64, 128
    mlp = fg.GroupedMlp(h, f, 2, torch.bfloat16, device=cuda)
    x = randn_bf16((64, h), 0).to(cuda)
    with torch.no_grad(), fg.fp8_autocast(enabled=True):
        y0 = mlp(x, torch.tensor(sizes))
    # frozen weights: only grad_input is produced, no transposes of the activations are needed
    for p in mlp.parameters():
        p.requires_grad_(False)
    xin = x.clone().requires_grad_(True)
    with fg.fp8_autocast(enabled=True):
        y1 = mlp(xin, torch.tensor(sizes))
    y1.sum().backward()
    assert xin.grad is not None and torch.isfinite(xin.grad.float()).all()
    assert y0.shape == y1.shape == (64, h)


def test_state_dict_round_trip_reproduces_fp8_state(cuda):
    import fp8_gmm_b200 as fg

    sizes, k, n = [40, 24], 64, 32
    a = fg.GroupedLinear(k, n, 2, torch.bfloat16, device=cuda)
    rec = fg.DelayedScaling(amax_history_len=4)
    for i in range(3):
        x = randn_bf16((64, k), i).to(cuda).requires_grad_(True)
        with fg.fp8_autocast(enabled=True, fp8_recipe=rec):
            a(x, torch.tensor(sizes)).sum().backward()
    state = copy.deepcopy(a.state_dict())
    b = fg.GroupedLinear(k, n, 2, torch.bfloat16, device=cuda)
    b.load_state_dict(state)
    x = randn_bf16((64, k), 9).to(cuda)
    outs = []
    for layer in (a, b):
        xin = x.clone().requires_grad_(True)
        layer.weight_tensor.grad = None
        with fg.fp8_autocast(enabled=True, fp8_recipe=rec):
            y = layer(xin, torch.tensor(sizes))
        y.sum().backward()
        outs.append((y.detach(), xin.grad, layer.weight_tensor.grad))
    for t0, t1 in zip(*outs):
        assert torch.equal(t0, t1)
    assert torch.equal(a.fp8_meta["scaling_fwd"].scale, b.fp8_meta["scaling_fwd"].scale)
    assert torch.equal(a.fp8_meta["scaling_bwd"].amax_history, b.fp8_meta["scaling_bwd"].amax_history)


def test_fine_grained_zipf_routing(cuda):
    """The fine-grained MoE shapes (E=64, hidden 2048, ffn 1408, Zipf loads with empty and ragged groups) at a
    reduced row count: outputs finite, empty experts get exactly zero weight gradients, and rows of
    each group depend only on that group's weights (zeroing another expert's weights changes nothing)."""
    import fp8_gmm_b200 as fg

    E, h, f = 64, 2048, 1408
    sizes = routed_group_sizes(E, 6144, seed=1, zipf_s=1.2)
    sizes[-2] += sizes[-1]  # make sure at least one expert receives no rows
    sizes[-1] = 0
    assert 0 in sizes and any(s % 16 for s in sizes)
    mlp = fg.GroupedMlp(h, f, E, torch.bfloat16, device=cuda, activation="swiglu")
    x = randn_bf16((sum(sizes), h), 0).to(cuda).requires_grad_(True)
    with fg.fp8_autocast(enabled=True):
        y = mlp(x, torch.tensor(sizes))
    y.backward(randn_bf16(tuple(y.shape), 1).to(cuda))
    fg.backend.device_status()
    assert torch.isfinite(y.float()).all() and torch.isfinite(x.grad.float()).all()
    for g, s in enumerate(sizes):
        if s == 0:
            assert (mlp.fc1_weight.grad[g] == 0).all() and (mlp.fc2_weight.grad[g] == 0).all()
    busiest = max(range(E), key=lambda g: sizes[g])
    other = (busiest + 1) % E
    with torch.no_grad():
        mlp.fc1_weight[other].zero_()
        mlp2 = copy.deepcopy(mlp)
    start = sum(sizes[:busiest])
    with torch.no_grad(), fg.fp8_autocast(enabled=True):
        # fresh metas for both modules so the scales are the same first-step ones
        a = fg.GroupedMlp(h, f, E, torch.bfloat16, device=cuda, activation="swiglu")
        a.load_state_dict({k: v for k, v in mlp2.state_dict().items() if "extra" not in k}, strict=False)
        y2 = a(x.detach(), torch.tensor(sizes))
    assert torch.equal(y2[start:start + sizes[busiest]], y.detach()[start:start + sizes[busiest]])


@pytest.mark.parametrize("act", ["gelu", "swiglu"])
def test_row_permutation_is_equivalent_to_gather_scatter(cuda, act):
    """Rows handed over in a block-permuted ("source-major") order, with the permutation applied by the cast and the
    GEMM epilogues, must give exactly what the plain module gives on expert-major rows, forward and backward."""
    import fp8_gmm_b200 as fg
    from fp8_gmm_b200 import ep
    from fp8_gmm_b200.backend import RowPermutation

    h, f, P, El = 128, 256, 3, 4
    g = torch.Generator().manual_seed(3)
    counts = torch.randint(0, 40, (P, El), generator=g)
    counts[1, 2] = 0
    sizes = counts.sum(0)
    m = int(sizes.sum())
    to_em, to_sm = ep.block_permutation(counts)
    src, dst, rows, grp = ep.permutation_blocks(counts)
    perm = RowPermutation(src, dst, rows, grp, to_em.to(torch.int32).to(cuda))
    x_sm = randn_bf16((m, h), 0)          # source-major rows, as an all-to-all would deliver them
    dy_sm = randn_bf16((m, h), 1)
    outs = []
    for use_perm in (True, False):
        torch.manual_seed(5)
        mlp = fg.GroupedMlp(h, f, El, torch.bfloat16, device=cuda, activation=act)
        xin = (x_sm if use_perm else x_sm[to_em]).to(cuda).requires_grad_(True)
        with fg.fp8_autocast(enabled=True):
            y = mlp(xin, sizes, row_permutation=perm if use_perm else None)
        y.backward((dy_sm if use_perm else dy_sm[to_em]).to(cuda))
        fg.backend.device_status()
        outs.append((y.detach().cpu(), xin.grad.cpu(), mlp.fc1_weight.grad.cpu(), mlp.fc2_weight.grad.cpu(),
                     mlp.fp8_meta["scaling_fwd"].amax_history[0].cpu(), mlp.fp8_meta["scaling_bwd"].amax_history[0].cpu()))
    (y_p, gx_p, gw1_p, gw2_p, af_p, ab_p), (y_e, gx_e, gw1_e, gw2_e, af_e, ab_e) = outs
    assert torch.equal(y_p[to_em], y_e) and torch.equal(gx_p[to_em], gx_e)
    assert torch.equal(gw1_p, gw1_e) and torch.equal(gw2_p, gw2_e)
    assert torch.equal(af_p, af_e) and torch.equal(ab_p, ab_e)


@pytest.mark.parametrize("kind", ["linear", "mlp"])
def test_weight_cache_across_microbatches(cuda, kind):
    """is_first_microbatch=True casts and keeps the FP8 weights, False reuses them: two micro-batches give the same
    results as with is_first_microbatch=None as long as the scales do not move in between (update interval 1000),
    the cached tensors are the very same objects, and the number of kernel launches drops by the weight casts."""
    import fp8_gmm_b200 as fg

    sizes, k, n = [40, 0, 24], 64, 128
    make = (lambda: fg.GroupedLinear(k, n, 3, torch.bfloat16, device=cuda)) if kind == "linear" else (
        lambda: fg.GroupedMlp(k, n, 3, torch.bfloat16, device=cuda, activation="swiglu"))
    torch.manual_seed(0)
    ref_layer = make()
    layer = make()
    layer.load_state_dict(copy.deepcopy(ref_layer.state_dict()))
    xs = [randn_bf16((64, k), 20 + i).to(cuda) for i in range(2)]
    results = {}
    for name, mod, flags in (("plain", ref_layer, [None, None]), ("cached", layer, [True, False])):
        outs, launches = [], []
        for x, flag in zip(xs, flags):
            xin = x.clone().requires_grad_(True)
            before = fg.backend.launch_count()
            with fg.fp8_autocast(enabled=True, fp8_recipe=fg.DelayedScaling(interval=1000, amax_history_len=4)):
                y = mod(xin, torch.tensor(sizes), is_first_microbatch=flag)
            launches.append(fg.backend.launch_count() - before)
            y.float().sum().backward()
            outs.append((y.detach().clone(), xin.grad.clone()))
        results[name] = (outs, launches, [p.grad.clone() for p in mod.parameters()])
    for (y0, g0), (y1, g1) in zip(results["plain"][0], results["cached"][0]):
        assert torch.equal(y0, y1) and torch.equal(g0, g1)
    for w0, w1 in zip(results["plain"][2], results["cached"][2]):
        assert torch.equal(w0, w1)
    n_weights = 1 if kind == "linear" else 2
    assert results["cached"][1][1] == results["plain"][1][1] - n_weights, results
    pad = layer.get_fp8_weights_scratchpad(False)
    # [fp8 weight, its transpose] per weight; the transposes only exist in the reference's dataflow (FP8GMM_DGRAD=transposed)
    assert all(t is not None and t.dtype == torch.float8_e4m3fn for t in pad[0::2])
    assert all(t is None or t.dtype == torch.float8_e4m3fn for t in pad[1::2])
    fg.backend.device_status()
