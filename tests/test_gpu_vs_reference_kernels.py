"""GPU: this package's elementwise kernels against the reference's own kernels on the same device.

The reference's csrc/multi_pointwise.cu and csrc/multi_pad_fusion.cu compile unmodified for sm_100a
(oracle/build_ref_kernels.py puts the extension into the git-ignored oracle/_ref/, which travels with
the working tree).  When that file is present this is the strongest pin there is: FP8 bytes, padding
layout and amax must be identical on the reference's full shape fixture (fp8_gmm/test.py:10-21).
Skipped when the extension has not been built.
"""
import glob
import importlib.util
import os

import pytest
import torch

from tests.helpers import FP8_DTYPES, REF_SHAPES, padded_rows, randn_bf16, u8

pytestmark = pytest.mark.gpu
_SO = glob.glob(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref",
                             "ref_fp8_gmm_kernels*.so"))


@pytest.fixture(scope="module")
def ref(cuda):
    if not _SO:
        pytest.skip("oracle/_ref/ref_fp8_gmm_kernels*.so not built")
    spec = importlib.util.spec_from_file_location("ref_fp8_gmm_kernels", _SO[0])
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _inputs(cuda, seed0):
    xs = [randn_bf16(s, seed0 + i).to(cuda) for i, s in enumerate(REF_SHAPES)]
    sc = [torch.tensor([0.3 + 1.1 * i], device=cuda) for i in range(len(xs))]
    return xs, sc


@pytest.mark.parametrize("dtype", FP8_DTYPES)
def test_quantize_identical(cuda, ref, dtype):
    from fp8_gmm_b200 import backend

    xs, sc = _inputs(cuda, 0)
    o1 = [torch.empty_like(x, dtype=dtype) for x in xs]
    o2 = [torch.empty_like(x, dtype=dtype) for x in xs]
    a1 = [torch.zeros(1, device=cuda) for _ in xs]
    a2 = [torch.zeros(1, device=cuda) for _ in xs]
    ref.multi_quantize(xs, o1, sc, a1)
    backend.multi_quantize(xs, o2, sc, a2)
    for p, q, a, b in zip(o1, o2, a1, a2):
        assert torch.equal(u8(p), u8(q)) and torch.equal(a, b)


@pytest.mark.parametrize("dtype", FP8_DTYPES)
@pytest.mark.parametrize("padded", [True, False])
def test_cast_transpose_and_transpose_identical(cuda, ref, dtype, padded):
    from fp8_gmm_b200 import backend

    xs, sc = _inputs(cuda, 100)
    mk_t = lambda: [torch.empty(s[1], padded_rows(s[0], padded), dtype=dtype, device=cuda) for s in REF_SHAPES]  # noqa: E731
    o1, o2 = [torch.empty_like(x, dtype=dtype) for x in xs], [torch.empty_like(x, dtype=dtype) for x in xs]
    t1, t2 = mk_t(), mk_t()
    a1 = [torch.zeros(1, device=cuda) for _ in xs]
    a2 = [torch.zeros(1, device=cuda) for _ in xs]
    ref.multi_pad_cast_transpose(xs, o1, t1, sc, a1)
    backend.multi_cast_transpose(xs, o2, t2, sc, a2)
    for i in range(len(xs)):
        assert torch.equal(u8(o1[i]), u8(o2[i])) and torch.equal(u8(t1[i]), u8(t2[i])) and torch.equal(a1[i], a2[i])
    r1, r2 = mk_t(), mk_t()
    ref.multi_pad_transpose(o1, r1)
    backend.multi_transpose(o1, r2)
    for p, q in zip(r1, r2):
        assert torch.equal(u8(p), u8(q))


def test_scale_mul_identical(cuda, ref):
    from fp8_gmm_b200 import backend

    xs, sc = _inputs(cuda, 200)
    ys = [x.clone() for x in xs]
    s2 = [torch.tensor([0.01 * (i + 1)], device=cuda) for i in range(len(xs))]
    ref.multi_scale_mul(xs, sc, s2)
    backend.multi_scale_mul(ys, sc, s2)
    for p, q in zip(xs, ys):
        assert torch.equal(p.view(torch.int16), q.view(torch.int16))


@pytest.mark.parametrize("dtype", FP8_DTYPES)
def test_dgelu_identical_or_within_one_step(cuda, ref, dtype):
    """Same expression and the same fast-math build flags: expected to be identical; the assertion allows
    one FP8 step on < 0.1 % of elements in case instruction selection differs."""
    from fp8_gmm_b200 import backend

    xs, sc = _inputs(cuda, 300)
    ps = [randn_bf16(s, 400 + i).to(cuda) for i, s in enumerate(REF_SHAPES)]
    mk_t = lambda: [torch.empty(s[1], padded_rows(s[0], True), dtype=dtype, device=cuda) for s in REF_SHAPES]  # noqa: E731
    o1, o2 = [torch.empty_like(x, dtype=dtype) for x in xs], [torch.empty_like(x, dtype=dtype) for x in xs]
    t1, t2 = mk_t(), mk_t()
    a1 = [torch.zeros(1, device=cuda) for _ in xs]
    a2 = [torch.zeros(1, device=cuda) for _ in xs]
    ref.multi_pad_cast_transpose_dgelu(xs, ps, o1, t1, sc, a1)
    backend.multi_cast_transpose_dgelu(xs, ps, o2, t2, sc, a2)
    worst = 0.0
    for i in range(len(xs)):
        diff = (u8(o1[i]).int() - u8(o2[i]).int()).abs()
        assert int(diff.max()) <= 1
        worst = max(worst, float((diff != 0).float().mean()))
        assert torch.equal(u8(t2[i])[:, : REF_SHAPES[i][0]], u8(o2[i]).t())
        assert abs(float(a1[i]) - float(a2[i])) <= 1e-3 * float(a1[i])
    print(f"dgelu {dtype}: worst mismatch fraction {worst:.2e}")
    assert worst < 1e-3
