"""GPU: the multi-tensor elementwise kernels against the CPU oracle, byte for byte.

Shapes are the reference's own test fixture (fp8_gmm/test.py:10-21), which straddles every boundary of
its aligned/unaligned launch split; the assertions are exact where the reference's tests use
atol=rtol=0.2 (fp8_gmm/test.py:36-101), because FP8 bytes, padding layout and amax are an integer
contract.  Scales are positive (a negative scale turns padding into -0; covered separately).
"""
import pytest
import torch

from oracle import oracle as O
from tests.helpers import FP8_DTYPES, REF_SHAPES, fp8_steps, padded_rows, randn_bf16, u8

pytestmark = pytest.mark.gpu


def _scales(n, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [float(torch.rand(1, generator=g) * 7 + 0.05) for _ in range(n)]


@pytest.mark.parametrize("dtype", FP8_DTYPES)
def test_multi_quantize_bit_exact(cuda, dtype):
    from fp8_gmm_b200 import backend

    xs = [randn_bf16(s, i) for i, s in enumerate(REF_SHAPES)]
    sc = _scales(len(xs))
    d_x = [x.to(cuda) for x in xs]
    d_out = [torch.empty_like(x, dtype=dtype) for x in d_x]
    d_sc = [torch.tensor([s], device=cuda) for s in sc]
    d_am = [torch.tensor([0.0], device=cuda) for _ in xs]
    backend.multi_quantize(d_x, d_out, d_sc, d_am)
    for x, s, o, a in zip(xs, sc, d_out, d_am):
        assert torch.equal(u8(o).cpu(), u8(O.quantize(x, torch.tensor(s), dtype)))
        assert float(a) == O.amax_merge(x)


def test_multi_quantize_amax_merges_and_handles_specials(cuda):
    from fp8_gmm_b200 import backend

    x = randn_bf16((300, 77), 5)
    x[0, 0], x[1, 1], x[2, 2] = float("nan"), float("inf"), -1e30
    d_x = x.to(cuda)
    out = torch.empty_like(d_x, dtype=torch.float8_e4m3fn)
    am = torch.tensor([1e38], device=cuda)
    backend.multi_quantize([d_x], [out], [torch.tensor([2.0], device=cuda)], [am])
    assert float(am) == float("inf")  # |inf| wins over the preloaded value, NaN is ignored
    assert torch.equal(u8(out).cpu(), u8(O.quantize(x, 2.0, torch.float8_e4m3fn)))
    # more tensors than the reference's per-call cap of 64 (csrc/multi_pointwise.cu:13), incl. empty ones
    xs = [randn_bf16((i % 7, 5 + i), i) for i in range(400)]
    d_xs = [t.to(cuda) for t in xs]
    outs = [torch.empty_like(t, dtype=torch.float8_e5m2) for t in d_xs]
    ams = torch.zeros(400, device=cuda)
    backend.multi_quantize(d_xs, outs, [None] * 400, [ams[i] for i in range(400)])
    for i in range(400):
        assert torch.equal(u8(outs[i]).cpu(), u8(O.quantize(xs[i], 1.0, torch.float8_e5m2)))
        assert float(ams[i]) == O.amax_merge(xs[i])


@pytest.mark.parametrize("dtype", FP8_DTYPES)
@pytest.mark.parametrize("padded", [True, False])
def test_multi_transpose_bit_exact(cuda, dtype, padded):
    from fp8_gmm_b200 import backend

    qs = [randn_bf16(s, i).to(dtype) for i, s in enumerate(REF_SHAPES)]
    d_q = [q.to(cuda) for q in qs]
    d_t = [torch.full((s[1], padded_rows(s[0], padded)), 0x55, dtype=torch.uint8, device=cuda).view(dtype) for s in REF_SHAPES]
    backend.multi_transpose(d_q, d_t)
    for q, t, s in zip(qs, d_t, REF_SHAPES):
        assert torch.equal(u8(t).cpu(), u8(O.pad_transpose(q, padded_rows(s[0], padded))))


@pytest.mark.parametrize("dtype", FP8_DTYPES)
@pytest.mark.parametrize("padded", [True, False])
def test_multi_cast_transpose_bit_exact(cuda, dtype, padded):
    from fp8_gmm_b200 import backend

    xs = [randn_bf16(s, 10 + i) for i, s in enumerate(REF_SHAPES)]
    sc = _scales(len(xs), 1)
    d_x = [x.to(cuda) for x in xs]
    d_o = [torch.empty_like(x, dtype=dtype) for x in d_x]
    d_t = [torch.empty(s[1], padded_rows(s[0], padded), dtype=dtype, device=cuda) for s in REF_SHAPES]
    d_sc = [torch.tensor([s], device=cuda) for s in sc]
    d_am = [torch.tensor([0.0], device=cuda) for _ in xs]
    backend.multi_cast_transpose(d_x, d_o, d_t, d_sc, d_am)
    for x, s, o, t, a, shape in zip(xs, sc, d_o, d_t, d_am, REF_SHAPES):
        q, qt, am = O.pad_cast_transpose(x, torch.tensor(s), dtype, padded_rows(shape[0], padded))
        assert torch.equal(u8(o).cpu(), u8(q))
        assert torch.equal(u8(t).cpu(), u8(qt))
        assert float(a) == am


def test_negative_scale_padding_is_minus_zero(cuda):
    from fp8_gmm_b200 import backend

    x = randn_bf16((21, 40), 3)
    o = torch.empty(21, 40, dtype=torch.float8_e4m3fn, device=cuda)
    t = torch.empty(40, 32, dtype=torch.float8_e4m3fn, device=cuda)
    backend.multi_cast_transpose([x.to(cuda)], [o], [t], [torch.tensor([-1.5], device=cuda)], [torch.zeros(1, device=cuda)])
    q, qt, _ = O.pad_cast_transpose(x, -1.5, torch.float8_e4m3fn, 32)
    assert torch.equal(u8(t).cpu(), u8(qt)) and torch.equal(u8(o).cpu(), u8(q))
    assert (u8(t).cpu()[:, 21:] == 0x80).all()


def _assert_within_fp8_steps(diff):
    """Fast-math tanh / exp on the GPU against the host's libm in the oracle: one FP8 step on under 2 % of the
    elements.  Where the product sits in the FP8 subnormal range (steps are absolute there) and the host's own
    tanh differs in the last bit between CPU generations, a single element in a few million may land two steps off."""
    assert int(diff.max()) <= 2, int(diff.max())
    assert float((diff > 1).float().mean()) < 1e-5 and float((diff != 0).float().mean()) < 2e-2


@pytest.mark.parametrize("dtype", FP8_DTYPES)
def test_multi_cast_transpose_dgelu_within_one_fp8_step(cuda, dtype):
    """The GPU evaluates tanh with the fast-math approximation (as the reference build does), the oracle
    with libm: bytes may differ by one FP8 step on a small fraction of elements; layout must be exact."""
    from fp8_gmm_b200 import backend

    shapes = [(768, 1024), (120, 2080), (8, 8), (1, 3221), (2333, 1), (1481, 677)]
    xs = [randn_bf16(s, 20 + i) for i, s in enumerate(shapes)]
    ps = [randn_bf16(s, 40 + i) for i, s in enumerate(shapes)]
    d_x, d_p = [x.to(cuda) for x in xs], [p.to(cuda) for p in ps]
    d_o = [torch.empty_like(x, dtype=dtype) for x in d_x]
    d_t = [torch.empty(s[1], padded_rows(s[0], True), dtype=dtype, device=cuda) for s in shapes]
    d_sc = [torch.tensor([3.0], device=cuda) for _ in xs]
    d_am = [torch.tensor([0.0], device=cuda) for _ in xs]
    backend.multi_cast_transpose_dgelu(d_x, d_p, d_o, d_t, d_sc, d_am)
    for x, p, o, t, a, shape in zip(xs, ps, d_o, d_t, d_am, shapes):
        q, qt, am = O.pad_cast_transpose(x, 3.0, dtype, padded_rows(shape[0], True), pre_act=p)
        diff = fp8_steps(o.cpu(), q)
        _assert_within_fp8_steps(diff)
        # transposed copy carries the very same bytes as the row-major copy, padding is zero
        assert torch.equal(u8(t).cpu()[:, : shape[0]], u8(o).cpu().t())
        assert (u8(t).cpu()[:, shape[0]:] == 0).all()
        assert abs(float(a) - am) <= 2e-3 * max(am, 1e-3)


@pytest.mark.parametrize("dtype", FP8_DTYPES)
def test_multi_cast_transpose_dswiglu(cuda, dtype):
    from fp8_gmm_b200 import backend

    shapes = [(256, 512), (130, 72), (7, 8), (33, 1408)]
    for i, (m, f) in enumerate(shapes):
        dy, h = randn_bf16((m, f), 60 + i), randn_bf16((m, 2 * f), 80 + i)
        pr = padded_rows(m, True)
        o = torch.empty(m, 2 * f, dtype=dtype, device=cuda)
        t = torch.empty(2 * f, pr, dtype=dtype, device=cuda)
        am = torch.zeros(1, device=cuda)
        backend.multi_cast_transpose_dswiglu([dy.to(cuda)], [h.to(cuda)], [o], [t], [torch.tensor([2.0], device=cuda)], [am])
        v = O.dswiglu(dy.float(), h.float())
        q = O.quantize(v, 2.0, dtype)
        diff = fp8_steps(o.cpu(), q)
        _assert_within_fp8_steps(diff)
        assert torch.equal(u8(t).cpu()[:, :m], u8(o).cpu().t()) and (u8(t).cpu()[:, m:] == 0).all()
        assert abs(float(am) - O.amax_merge(v)) <= 2e-3 * O.amax_merge(v)


def test_multi_scale_mul_bit_exact(cuda):
    from fp8_gmm_b200 import backend

    xs = [randn_bf16(s, 90 + i) for i, s in enumerate(REF_SHAPES[4:] + [(512, 1024)])]
    d_x = [x.to(cuda) for x in xs]
    s1 = [torch.tensor([0.013 * (i + 1)], device=cuda) for i in range(len(xs))]
    s2 = [torch.tensor([1.7 / (i + 1)], device=cuda) for i in range(len(xs))]
    backend.multi_scale_mul(d_x, s1, s2)
    for x, a, b, got in zip(xs, s1, s2, d_x):
        assert torch.equal(got.cpu().view(torch.int16), O.scale_mul(x, float(a), float(b)).view(torch.int16))


def test_grouped_form_matches_list_form(cuda):
    """The grouped C-ABI entry point writes the same bytes as the list form on per-group views."""
    from fp8_gmm_b200 import backend
    from fp8_gmm_b200.utils import cumsum_group_sizes

    sizes = [128, 0, 37, 300, 16, 1]
    G, padded, cums, pcs = cumsum_group_sizes(sizes, need_padding=True)
    k = 192
    x = randn_bf16((cums[-1], k), 7)
    d_x = x.to(cuda)
    scale = torch.rand(3 * G, device=cuda) + 0.5
    amax = torch.zeros(3 * G, device=cuda)
    out = torch.empty(cums[-1], k, dtype=torch.float8_e4m3fn, device=cuda)
    out_t = torch.empty(pcs[-1], k, dtype=torch.float8_e4m3fn, device=cuda)
    backend.grouped_cast_transpose(d_x, cums, out, out_t, pcs, (scale, 3), (amax, 3))
    for g in range(G):
        q, qt, am = O.pad_cast_transpose(x[cums[g]:cums[g + 1]], scale[3 * g].cpu(), torch.float8_e4m3fn, pcs[g + 1] - pcs[g])
        assert torch.equal(u8(out[cums[g]:cums[g + 1]]).cpu(), u8(q))
        blk = u8(out_t)[pcs[g]:pcs[g + 1]].reshape(k, pcs[g + 1] - pcs[g]) if pcs[g + 1] > pcs[g] else None
        if blk is not None:
            assert torch.equal(blk.cpu(), u8(qt))
        assert float(amax[3 * g]) == am
    assert float(amax[1]) == 0.0 and float(amax[2]) == 0.0  # neighbouring slots untouched
    # pure fp8 transpose through the grouped form
    t2 = torch.empty_like(out_t)
    backend.grouped_cast_transpose(out, cums, None, t2, pcs, None, None)
    assert torch.equal(u8(t2).cpu(), u8(out_t).cpu())


def test_delayed_scaling_update_kernel(cuda):
    from fp8_gmm_b200 import backend

    g = torch.Generator().manual_seed(0)
    hist = torch.rand(16, 40, generator=g) * 10
    hist[3, 5] = float("inf")
    hist[:, 7] = 0
    scale = torch.rand(40, generator=g) + 1
    for algo in ("max", "most_recent"):
        for margin in (0, 2):
            d_h, d_s, d_i = hist.to(cuda), scale.to(cuda), torch.empty(40, device=cuda)
            backend.delayed_scaling_update(d_h, d_s, d_i, 448.0, margin, algo)
            nh, ns, ni = O.delayed_scaling_update(hist, scale, 448.0, margin, algo)
            assert torch.equal(d_h.cpu(), nh) and torch.equal(d_s.cpu(), ns) and torch.equal(d_i.cpu(), ni)


@pytest.mark.parametrize("width,dtype", [(4096, torch.float8_e4m3fn), (256, torch.bfloat16), (16, torch.uint8)])
def test_block_permute_rows_moves_runs_of_rows(cuda, width, dtype):
    """fp8gmm_block_permute_rows: runs of consecutive rows copied to new row positions (the expert-parallel forward
    uses it to bring rows that arrived source-major into expert-major order).  Exact copy; rows outside every block
    stay untouched; empty blocks and more blocks than one launch carries are handled."""
    from fp8_gmm_b200 import backend

    g = torch.Generator().manual_seed(width)
    counts = torch.randint(0, 40, (200,), generator=g)
    counts[5] = 0
    total = int(counts.sum())
    src_start = (torch.cumsum(counts, 0) - counts).tolist()
    order = torch.randperm(len(counts), generator=g)
    dst_start = torch.empty(len(counts), dtype=torch.int64)
    pos = 3                                                     # three leading rows of dst belong to no block
    for b in order.tolist():
        dst_start[b] = pos
        pos += int(counts[b])
    raw = torch.randint(0, 256, (total, width * torch.empty((), dtype=dtype).element_size()), generator=g, dtype=torch.uint8)
    src = raw.to(cuda).view(dtype)
    dst = torch.full((total + 3, raw.shape[1]), 0x5A, dtype=torch.uint8, device=cuda).view(dtype)
    backend.block_permute_rows(src, dst, src_start, dst_start.tolist(), counts.tolist())
    backend.device_status()
    got = dst.view(torch.uint8).cpu()
    assert (got[:3] == 0x5A).all()
    for b in range(len(counts)):
        n = int(counts[b])
        assert torch.equal(got[int(dst_start[b]):int(dst_start[b]) + n], raw[src_start[b]:src_start[b] + n])
