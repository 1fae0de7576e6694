"""CPU: pin the oracle before trusting it.

1. the plain-C converter against the CUDA toolkit's host-side __nv_fp8_e4m3/__nv_fp8_e5m2 constructors
   (the converter the reference's kernels call, reference csrc/utils.cuh:11-12) over every bf16 bit
   pattern times several scales, and over random fp32 values;
2. the torch restatement (oracle/oracle.py) against the C restatement (oracle/fp8_oracle.c) for
   quantise, amax, padded transposes, dGELU cast and the GEMM;
3. both against the committed golden vectors in tests/golden/ that were produced on a B200 by the
   reference's own kernels (tests/golden/make_golden.py), when present.
"""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import c_oracle as C
from oracle import oracle as O
from tests.helpers import padded_rows, randn_bf16, u8

FMT = {torch.float8_e4m3fn: 0, torch.float8_e5m2: 1}


def bf16_u16(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


@pytest.mark.parametrize("scale", [1.0, 0.37, 448 / 3.3, 57344 / 2.9, 1e-3, 1e4, -2.5])
@pytest.mark.parametrize("dtype", list(FMT))
def test_converters_agree_on_every_bf16_value(scale, dtype):
    bits = np.arange(65536, dtype=np.uint16)
    x = (bits.astype(np.uint32) << 16).view(np.float32)
    with np.errstate(all="ignore"):
        y = (x * np.float32(scale)).astype(np.float32)
    ref = C.toolkit_cvt(y, FMT[dtype])
    assert np.array_equal(C.cvt_array(y, FMT[dtype]), ref)
    t = O.quantize(torch.from_numpy(bits.view(np.int16)).view(torch.bfloat16), scale, dtype)
    assert np.array_equal(u8(t).numpy(), ref)


@pytest.mark.parametrize("dtype", list(FMT))
def test_converters_agree_on_random_fp32(dtype):
    rng = np.random.default_rng(0)
    x = (rng.standard_normal(500_000) * np.exp(rng.uniform(-25, 14, 500_000))).astype(np.float32)
    x[:8] = [0.0, -0.0, np.inf, -np.inf, np.nan, 448.0, 464.0, 61440.0]
    assert np.array_equal(C.cvt_array(x, FMT[dtype]), C.toolkit_cvt(x, FMT[dtype]))


def test_saturation_and_ties():
    e4, e5 = 0, 1
    cases = np.array([448.0, 463.9, 464.0, 465.0, 1e9, -1e9, 2**-9, 2**-10, 2**-10 * 1.01], dtype=np.float32)
    assert list(C.cvt_array(cases, e4)) == [0x7E, 0x7E, 0x7E, 0x7E, 0x7E, 0xFE, 0x01, 0x00, 0x01]
    cases5 = np.array([57344.0, 61439.0, 61440.0, 1e9, 2**-16, 2**-17], dtype=np.float32)
    assert list(C.cvt_array(cases5, e5)) == [0x7B, 0x7B, 0x7B, 0x7B, 0x01, 0x00]


@pytest.mark.parametrize("shape", [(8, 8), (1, 321), (233, 1), (120, 208), (148, 67)])
@pytest.mark.parametrize("dtype", list(FMT))
@pytest.mark.parametrize("padded", [True, False])
def test_torch_and_c_restatements_agree(shape, dtype, padded):
    x = randn_bf16(shape, seed=sum(shape))
    scale = 3.7
    pr = padded_rows(shape[0], padded)
    q, qt, am = O.pad_cast_transpose(x, scale, dtype, pr, prev_amax=0.25)
    cq, cqt, cam = C.pad_cast_transpose(bf16_u16(x), scale, FMT[dtype], pr, amax0=0.25)
    assert np.array_equal(u8(q).numpy(), cq) and np.array_equal(u8(qt).numpy(), cqt)
    assert am == cam
    # flat quantise gives the same bytes
    fq, fam = C.quantize(bf16_u16(x), scale, FMT[dtype])
    assert np.array_equal(fq, cq) and fam == O.amax_merge(x)
    # pure transpose
    assert np.array_equal(u8(O.pad_transpose(q, pr)).numpy(), C.pad_transpose(cq, pr))


def test_negative_scale_pads_with_minus_zero():
    x = randn_bf16((5, 3), seed=1)
    q, qt, _ = O.pad_cast_transpose(x, -1.5, torch.float8_e4m3fn, 16)
    assert (u8(qt)[:, 5:] == 0x80).all()
    _, cqt, _ = C.pad_cast_transpose(bf16_u16(x), -1.5, 0, 16)
    assert np.array_equal(u8(qt).numpy(), cqt)


def test_dgelu_cast_restatements_agree_within_one_ulp():
    # libm tanhf (C) and torch.tanh may differ in the last fp32 bit: allow one fp8 step on rare elements
    x, pre = randn_bf16((64, 48), 3), randn_bf16((64, 48), 4)
    q, _, am = O.pad_cast_transpose(x, 2.0, torch.float8_e5m2, 64, pre_act=pre)
    cq, _, cam = C.pad_cast_transpose(bf16_u16(x), 2.0, 1, 64, gelu_in=bf16_u16(pre))
    diff = np.abs(u8(q).numpy().astype(np.int32) - cq.astype(np.int32))
    assert diff.max() <= 1 and (diff != 0).mean() < 1e-2
    assert abs(am - cam) <= 1e-6 * max(am, 1.0)


def test_scale_mul_and_gemm_restatements_agree():
    x = randn_bf16((40, 24), 7)
    got = C.scale_mul(bf16_u16(x), 0.3, 1.7)
    assert np.array_equal(got, bf16_u16(O.scale_mul(x, 0.3, 1.7)))
    a = O.quantize(randn_bf16((24, 32), 8), 8.0, torch.float8_e5m2)
    b = O.quantize(randn_bf16((16, 32), 9), 8.0, torch.float8_e4m3fn)
    c = C.gemm_nt(u8(a).numpy(), 1, u8(b).numpy(), 0, 1 / 64.0)
    ref = O.grouped_gemm(a, b[None], [24], [1 / 8.0], [1 / 8.0])
    # summation order differs (sequential C loop vs BLAS): compare as numbers, tightly
    got = torch.from_numpy(c.view(np.int16)).view(torch.bfloat16)
    assert O.rel_frobenius(got, ref) < 4e-3


def test_delayed_scaling_recipe():
    hist = torch.tensor([[1.0, 0.0, 5.0], [2.0, 0.0, float("inf")], [0.5, 0.0, 1.0]])
    scale = torch.tensor([3.0, 7.0, 9.0])
    new_hist, sf, inv = O.delayed_scaling_update(hist, scale, 448.0, margin=1, algo="max")
    assert torch.equal(sf, torch.tensor([448.0 / 2.0 / 2.0, 7.0, 9.0]))  # zero / inf amax keep the old scale
    assert torch.equal(inv, 1.0 / sf)
    assert torch.equal(new_hist, torch.tensor([[0.0, 0.0, 0.0], [0.5, 0.0, 1.0], [1.0, 0.0, 5.0]]))
    _, sf2, _ = O.delayed_scaling_update(hist, scale, 448.0, algo="most_recent")
    assert torch.equal(sf2, torch.tensor([448.0, 7.0, 448.0 / 5.0]))


GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "ref_kernels_*.npz")))


@pytest.mark.skipif(not GOLDEN, reason="no golden vectors committed yet")
@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p) for p in GOLDEN])
def test_oracle_reproduces_reference_kernel_outputs(path):
    """Golden vectors = outputs of the reference's own CUDA kernels on a B200 (see make_golden.py)."""
    z = np.load(path)
    dtype = torch.float8_e4m3fn if int(z["fmt"]) == 0 else torch.float8_e5m2
    x = torch.from_numpy(z["x"].view(np.int16)).view(torch.bfloat16)
    scale, pr = float(z["scale"]), int(z["padded_rows"])
    q, qt, am = O.pad_cast_transpose(x, scale, dtype, pr)
    assert np.array_equal(u8(q).numpy(), z["cast"])
    assert np.array_equal(u8(qt).numpy(), z["cast_t"])
    assert np.float32(am) == z["amax"]
    assert np.array_equal(u8(O.quantize(x, scale, dtype)).numpy(), z["quant"])
    assert np.array_equal(u8(O.pad_transpose(q, pr)).numpy(), z["transpose"])
    cq, cqt, cam = C.pad_cast_transpose(z["x"], scale, int(z["fmt"]), pr)
    assert np.array_equal(cq, z["cast"]) and np.array_equal(cqt, z["cast_t"]) and np.float32(cam) == z["amax"]
    assert np.array_equal(bf16_u16(O.scale_mul(x, float(z["s1"]), float(z["s2"]))), z["scale_mul"])
    if "dgelu_cast" in z:
        pre = torch.from_numpy(z["pre"].view(np.int16)).view(torch.bfloat16)
        dq, _, dam = O.pad_cast_transpose(x, scale, dtype, pr, pre_act=pre)
        diff = np.abs(u8(dq).numpy().astype(np.int32) - z["dgelu_cast"].astype(np.int32))
        # the reference evaluates tanh with the GPU's fast-math approximation: one fp8 step on rare elements
        assert diff.max() <= 1 and (diff != 0).mean() < 2e-2
        assert abs(dam - float(z["dgelu_amax"])) <= 2e-3 * max(dam, 1e-3)
