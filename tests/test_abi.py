"""CPU: the C-ABI library loads, exports every symbol the header declares, and rejects bad arguments
before touching the GPU (no compute call is made here)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_functions():
    text = open(os.path.join(ROOT, "include", "fp8_gmm_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fp8gmm_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = header_functions()
    for required in ["fp8gmm_multi_quantize", "fp8gmm_multi_scale_mul", "fp8gmm_multi_pad_transpose",
                     "fp8gmm_multi_pad_cast_transpose", "fp8gmm_multi_pad_cast_transpose_dgelu",
                     "fp8gmm_grouped_gemm", "fp8gmm_grouped_wgrad", "fp8gmm_last_error"]:
        assert required in names


def test_library_exports_every_declared_symbol():
    from fp8_gmm_b200 import _lib

    for name in header_functions():
        assert hasattr(_lib.lib, name), f"{name} is declared in the header but not exported"
        assert name in _lib.SYMBOLS, f"{name} has no ctypes prototype"
    assert _lib.lib.fp8gmm_version() >= 1000


def test_struct_layouts_match_the_header():
    """Field order and count of the ctypes mirrors follow the header's structs."""
    from fp8_gmm_b200 import _lib

    text = open(os.path.join(ROOT, "include", "fp8_gmm_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    for cname, cls in [("fp8gmm_tensor_desc", _lib.TensorDesc), ("fp8gmm_scale_mul_desc", _lib.ScaleMulDesc),
                       ("fp8gmm_grouped_cast_args", _lib.GroupedCastArgs), ("fp8gmm_gemm_args", _lib.GemmArgs),
                       ("fp8gmm_wgrad_args", _lib.WgradArgs)]:
        body = re.search(r"typedef struct \{([^{}]*)\}\s*" + cname + ";", text).group(1)
        fields = [re.search(r"(\w+)\s*$", f.strip()).group(1) for f in body.split(";") if f.strip()]
        mirror = [f[0].rstrip("_") for f in cls._fields_]
        assert fields == mirror, (cname, fields, mirror)


def test_bad_arguments_are_rejected_with_a_message():
    from fp8_gmm_b200 import _lib

    lib = _lib.lib
    assert lib.fp8gmm_multi_quantize(None, 3, 0, None) == 1
    assert b"descriptor" in lib.fp8gmm_last_error()
    d = (_lib.TensorDesc * 1)()
    assert lib.fp8gmm_multi_quantize(d, 1, 7, None) == 1
    assert b"format" in lib.fp8gmm_last_error()
    g = _lib.GemmArgs()
    g.num_groups, g.n, g.k = 1, 24, 32  # N not a multiple of 16
    assert lib.fp8gmm_grouped_gemm(ctypes.byref(g), None) == 1
    assert b"multiples of 16" in lib.fp8gmm_last_error()
    g.n = 32
    g.num_groups = 100000
    assert lib.fp8gmm_grouped_gemm(ctypes.byref(g), None) == 1
    w = _lib.WgradArgs()
    w.num_groups, w.n, w.k = 2, 32, 32
    offs = (ctypes.c_int64 * 3)(0, 16, 40)
    w.t_offsets = ctypes.cast(offs, ctypes.POINTER(ctypes.c_int64))
    w.c = 16
    w.a_scale_inv = w.b_scale_inv = 16
    assert lib.fp8gmm_grouped_wgrad(ctypes.byref(w), None) == 1  # no workspace
    assert b"workspace" in lib.fp8gmm_last_error()
    assert lib.fp8gmm_wgrad_workspace_bytes(8) == 8 * 2 * 128
    with pytest.raises(RuntimeError, match="status 1"):
        _lib.check(1, "demo")


def test_python_surface_matches_the_reference_names():
    import inspect

    import fp8_gmm_b200 as pkg
    from fp8_gmm_b200 import backend, utils

    sig = lambda f: list(inspect.signature(f).parameters)  # noqa: E731
    # reference fp8_gmm/backend.py:9,13,17,21,26,58-71
    assert sig(backend.multi_quantize) == ["inputs", "outputs", "scales", "amaxes"]
    assert sig(backend.multi_transpose) == ["inputs", "outputs"]
    assert sig(backend.multi_cast_transpose) == ["inputs", "outputs", "trans_outputs", "scales", "amaxes"]
    assert sig(backend.multi_cast_transpose_dgelu) == ["inputs", "gelu_inputs", "outputs", "trans_outputs", "scales", "amaxes"]
    assert sig(backend.cublas_fp8_gemm) == ["a", "b", "c", "a_scale_inv", "b_scale_inv", "pre_gelu_out", "c_scale", "c_amax", "backward"]
    assert sig(backend.fp8_gmm)[:12] == ["a", "b", "group_sizes", "a_scale_invs", "b_scale_invs", "c", "c_dtype",
                                         "pre_gelu_out", "c_scales", "c_amaxes", "backward", "cutlass"]
    # reference fp8_gmm/grouped_linear.py:187,204 and fp8_gmm/grouped_mlp.py:329,347
    assert sig(pkg.GroupedLinear.__init__)[1:] == ["in_features", "out_features", "num_groups", "dtype", "device", "cutlass"]
    assert sig(pkg.GroupedLinear.forward)[1:] == ["input", "group_sizes", "is_first_microbatch"]
    assert sig(pkg.GroupedMlp.__init__)[1:6] == ["in_features", "out_features", "num_groups", "dtype", "device"]
    assert sig(pkg.GroupedMlp.forward)[1:6] == ["input", "group_sizes", "has_tp", "tp_group", "is_first_microbatch"]
    assert pkg.GroupedMLP is pkg.GroupedMlp
    for name in ["MetaTensorType", "Fp8TensorType", "to_tex_dtype", "to_torch_dtype", "cumsum_group_sizes", "Fp8MetaWrapper"]:
        assert hasattr(utils, name)
