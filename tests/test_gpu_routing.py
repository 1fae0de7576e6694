"""GPU: router-side sort / gather / scatter (fp8_gmm_b200.routing) against the CPU restatement in oracle/oracle.py,
bit-exact for the integer outputs and the copies, and through autograd for the gradients."""
import pytest
import torch

from oracle import oracle as O
from tests.helpers import randn_bf16

pytestmark = pytest.mark.gpu


def _ids(tokens, top_k, E, seed):
    g = torch.Generator().manual_seed(seed)
    scores = torch.randn(tokens, E, generator=g)
    if E > 3:
        scores[:, 2] = -1e9  # an expert nobody picks
    return torch.topk(scores, top_k).indices.reshape(-1)


@pytest.mark.parametrize("tokens,top_k,E", [(1000, 2, 8), (4096, 8, 128), (37, 1, 4), (5000, 6, 64), (0, 2, 4)])
def test_sort_matches_stable_sort(cuda, tokens, top_k, E):
    from fp8_gmm_b200 import routing

    ids = _ids(tokens, top_k, E, 1)
    r = routing.sort_by_expert(ids.to(cuda), E)
    indices, bin_ids, bins, hist, inverse = O.moe_sort(ids, E)
    assert torch.equal(r.indices.cpu().long(), indices)
    assert torch.equal(r.bin_ids.cpu().long(), bin_ids)
    assert torch.equal(r.bins.cpu(), bins) and torch.equal(r.tokens_per_expert.cpu(), hist)
    assert torch.equal(r.inverse.cpu().long(), inverse)


@pytest.mark.parametrize("tokens,top_k,E,H", [(512, 2, 8, 256), (300, 8, 32, 136), (64, 3, 4, 33)])
def test_gather_scatter_match_oracle(cuda, tokens, top_k, E, H):
    from fp8_gmm_b200 import routing

    ids = _ids(tokens, top_k, E, 2)
    x = randn_bf16((tokens, H), 3)
    w = torch.rand(tokens, top_k, generator=torch.Generator().manual_seed(4))
    indices, bin_ids, bins, hist = routing.indices_and_bins(ids.to(cuda), E)
    o_idx, _, _, _, o_inv = O.moe_sort(ids, E)
    rows = routing.gather(x.to(cuda), indices, bin_ids, bins, top_k)
    assert torch.equal(rows.cpu(), O.moe_gather(x, o_idx, top_k))
    y = randn_bf16((tokens * top_k, H), 5)
    out = routing.scatter(y.to(cuda), indices, bin_ids, w.to(cuda), bins, top_k)
    assert torch.equal(out.cpu(), O.moe_scatter(y, o_inv, top_k, w))
    out1 = routing.scatter(y.to(cuda), indices, bin_ids, None, bins, top_k)
    assert torch.equal(out1.cpu(), O.moe_scatter(y, o_inv, top_k, None))


def test_gradients_match_a_torch_formulation(cuda):
    from fp8_gmm_b200 import routing

    tokens, top_k, E, H = 256, 2, 8, 128
    ids = _ids(tokens, top_k, E, 6).to(cuda)
    indices, bin_ids, bins, _ = routing.indices_and_bins(ids, E)
    x = randn_bf16((tokens, H), 7).to(cuda).requires_grad_(True)
    w = torch.rand(tokens, top_k, generator=torch.Generator().manual_seed(8)).to(cuda).requires_grad_(True)
    dy = randn_bf16((tokens, H), 9).to(cuda)
    rows = routing.gather(x, indices, bin_ids, bins, top_k)
    out = routing.scatter(rows * 1.5, indices, bin_ids, w, bins, top_k)
    out.backward(dy)
    # the same block in plain torch (fp32)
    xr = x.detach().float().requires_grad_(True)
    wr = w.detach().clone().requires_grad_(True)
    rows_r = xr[(indices.long() // top_k)] * 1.5
    inv = torch.empty_like(indices, dtype=torch.int64)
    inv[indices.long()] = torch.arange(indices.numel(), device=cuda)
    out_r = (wr.reshape(-1, 1) * rows_r[inv]).reshape(tokens, top_k, H).sum(1)
    out_r.backward(dy.float())
    assert torch.allclose(out.float(), out_r, rtol=2e-2, atol=2e-2)
    assert torch.allclose(x.grad.float(), xr.grad, rtol=3e-2, atol=3e-2)
    assert torch.allclose(w.grad, wr.grad, rtol=3e-2, atol=0.3)


def test_moe_block_like_the_reference_example(cuda):
    """Router -> sort -> gather -> GroupedMlp -> scatter, the dataflow of the reference's Fp8MlpModule
    (fp8_gmm/example.py:97-131) with this package's routing in place of megablocks."""
    import fp8_gmm_b200 as fg
    from fp8_gmm_b200 import routing

    tokens, H, F, E, top_k = 384, 128, 256, 8, 2
    torch.manual_seed(0)
    gate = torch.nn.Linear(H, E, bias=False).to(torch.bfloat16).to(cuda)
    mlp = fg.GroupedMlp(H, F, E, torch.bfloat16, device=cuda)
    x = randn_bf16((tokens, H), 11).to(cuda).requires_grad_(True)
    weights = torch.softmax(gate(x).float(), dim=1)
    multiplier, selected = torch.topk(weights, top_k)
    with torch.no_grad():
        indices, bin_ids, bins, tokens_per_expert = routing.indices_and_bins(selected.flatten(), E)
    rows = routing.gather(x, indices, bin_ids, bins, top_k)
    with fg.fp8_autocast(enabled=True):
        y = mlp(rows, tokens_per_expert.cpu().to(torch.long))
    out = routing.scatter(y, indices, bin_ids, multiplier.flatten(), bins, top_k)
    out.float().sum().backward()
    fg.backend.device_status()
    assert out.shape == (tokens, H) and torch.isfinite(out.float()).all()
    assert torch.isfinite(x.grad.float()).all() and x.grad.abs().sum() > 0
    assert gate.weight.grad is not None and torch.isfinite(gate.weight.grad.float()).all()
    assert mlp.fc1_weight.grad is not None


@pytest.mark.parametrize("tokens,E,top_k,renorm,dtype", [
    (2048, 8, 2, False, torch.float32),      # the reference example's router: top-2 of 8
    (2048, 8, 2, True, torch.float32),
    (333, 16, 1, False, torch.bfloat16),
    (1024, 128, 8, True, torch.float32),     # the expert-parallel workload's router
    (100, 64, 6, False, torch.bfloat16),
    (17, 1000, 40, True, torch.float32),     # more picks than a warp has lanes
])
def test_topk_router_matches_oracle(cuda, tokens, E, top_k, renorm, dtype):
    """softmax (fp32) + top-k + optional renormalisation as in the reference example (fp8_gmm/example.py:14-23).
    Weights within 2e-6 relative (the warp's summation order differs from torch's); expert ids exact wherever no two
    of the probabilities involved are within rounding of each other (equal logits may be named in either order)."""
    from fp8_gmm_b200 import routing

    g = torch.Generator().manual_seed(tokens + E)
    scores = (torch.randn(tokens, E, generator=g) * 2.0).to(dtype)
    want_w, want_e = O.moe_topk(scores, top_k, renorm)
    got_w, got_e = routing.topk(scores.to(cuda), top_k, renorm)
    assert got_w.dtype == torch.float32 and got_e.dtype == torch.int64
    probs = torch.softmax(scores.float(), 1)
    # the weights are the k largest probabilities whichever of several equal experts is named (bf16 logits tie often)
    assert torch.allclose(got_w.cpu(), want_w, rtol=2e-6, atol=1e-9)
    picked = probs.gather(1, got_e.cpu())
    if renorm:
        picked = picked / picked.sum(1, keepdim=True)
    assert torch.allclose(picked, got_w.cpu(), rtol=2e-6, atol=1e-9)          # ids and weights belong together
    assert all(len(set(row)) == top_k for row in got_e.cpu().tolist())        # distinct experts per token
    srt = probs.sort(1, descending=True).values
    gaps = (srt[:, :-1] - srt[:, 1:])[:, :top_k].min(1).values          # smallest gap among the picks and the runner-up
    clear = gaps > 1e-6 * srt[:, 0]
    assert torch.equal(got_e.cpu()[clear], want_e[clear])               # no ties: the ids are determined
    if renorm:
        assert torch.allclose(got_w.sum(1).cpu(), torch.ones(tokens), atol=1e-6)


def test_topk_router_gradient(cuda):
    from fp8_gmm_b200 import routing

    g = torch.Generator().manual_seed(9)
    scores = torch.randn(64, 8, generator=g)
    up = torch.randn(64, 2, generator=g)
    for renorm in (False, True):
        s_ref = scores.clone().requires_grad_(True)
        w_ref, _ = O.moe_topk(s_ref, 2, renorm)
        (w_ref * up).sum().backward()
        s = scores.to(cuda).requires_grad_(True)
        w, _ = routing.topk(s, 2, renorm)
        (w * up.to(cuda)).sum().backward()
        assert torch.allclose(s.grad.cpu(), s_ref.grad, rtol=1e-4, atol=1e-6)


def test_invalid_expert_id_is_reported_not_dereferenced(cuda):
    """One id outside [0, num_experts): the sort reports it through the status word, leaves the row out of the
    permutation, and gather / scatter skip the unset entries instead of using them as row numbers."""
    from fp8_gmm_b200 import _lib, backend, routing

    E, top_k, tokens, H = 4, 2, 50, 64
    ids = _ids(tokens, top_k, E, 5)
    ids[11] = 9
    backend.device_status()
    r = routing.sort_by_expert(ids.to(cuda), E)
    assert _lib.lib.fp8gmm_device_status(torch.cuda.current_stream().cuda_stream) == 4
    assert int(r.bins[-1]) == tokens * top_k - 1
    assert int(r.inverse[11]) == -1 and int(r.indices[-1]) == -1
    x = randn_bf16((tokens, H), 6).to(cuda)
    rows = routing.gather(x, r.indices, r.bin_ids, r.bins, top_k)
    back = routing.scatter(rows, r.indices, r.bin_ids, None, r.bins, top_k)
    torch.cuda.synchronize()
    assert _lib.lib.fp8gmm_device_status(torch.cuda.current_stream().cuda_stream) == 4
    keep = torch.ones(tokens, dtype=torch.bool)
    keep[11 // top_k] = False
    want = (x.float() * top_k).to(torch.bfloat16)
    assert torch.equal(back[keep.to(cuda)], want[keep.to(cuda)])      # every other token is untouched by the bad id
    backend.device_status()
