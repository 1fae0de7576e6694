"""Enums, dtype maps and FP8-meta bookkeeping of the reference's fp8_gmm/utils.py, same names.

`tex.DType` (Transformer Engine) is replaced by the small `DType` enum below because Transformer
Engine is not a dependency of this package; values with the same names map to the same torch dtypes.
"""
from enum import IntEnum

import torch


class DType(IntEnum):
    """Stand-in for ``transformer_engine ... tex.DType`` (reference fp8_gmm/utils.py:26-45)."""

    kFloat8E4M3 = 0
    kFloat8E5M2 = 1
    kBFloat16 = 2


# value passed to the C ABI (include/fp8_gmm_b200.h: fp8gmm_format)
FP8_FORMAT_CODE = {torch.float8_e4m3fn: 0, torch.float8_e5m2: 1}


class MetaTensorType(IntEnum):
    kScale = 0
    kScaleInv = 1
    kAmax = 2


class Fp8TensorType(IntEnum):
    kInputGroup1 = 0
    kInputGroup2 = 1
    kWeightGroup1 = 2
    kWeightGroup2 = 3
    kGradOutputGroup1 = 4
    kGradOutputGroup2 = 5
    kForwardInputGroup1 = 6
    kForwardInputGroup2 = 7
    kForwardWeightGroup1 = 8
    kForwardWeightGroup2 = 9


def to_tex_dtype(dtype):
    if dtype == torch.float8_e4m3fn:
        return DType.kFloat8E4M3
    if dtype == torch.float8_e5m2:
        return DType.kFloat8E5M2
    if dtype == torch.bfloat16:
        return DType.kBFloat16
    raise ValueError(f"Unsupported dtype: {dtype}")


def to_torch_dtype(dtype):
    if dtype == DType.kFloat8E4M3:
        return torch.float8_e4m3fn
    if dtype == DType.kFloat8E5M2:
        return torch.float8_e5m2
    if dtype == DType.kBFloat16:
        return torch.bfloat16
    raise ValueError(f"Unsupported dtype: {dtype}")


def cumsum_group_sizes(group_sizes, need_padding=False):
    """Prefix sums of the group sizes and, with ``need_padding``, of the sizes rounded up to 16 rows.

    Same contract as reference fp8_gmm/utils.py:48-62: returns (num_groups, padded, cumsums,
    padded_cumsums); ``padded`` says whether any group needed rounding, ``padded_cumsums`` is None
    without ``need_padding``.  The rounded sizes define the layout of the transposed FP8 buffers that
    feed the weight-gradient GEMM.
    """
    num_groups = len(group_sizes)
    padded = False
    cumsums = [0] * (num_groups + 1)
    padded_cumsums = [0] * (num_groups + 1) if need_padding else None
    for i, size in enumerate(group_sizes):
        size = int(size)
        cumsums[i + 1] = cumsums[i] + size
        if need_padding:
            rounded = (size + 15) // 16 * 16
            padded = padded or rounded != size
            padded_cumsums[i + 1] = padded_cumsums[i] + rounded
    return num_groups, padded, cumsums, padded_cumsums


class Fp8MetaWrapper:
    """Maps (tensor kind, group) to a slot of the recipe's meta vectors (reference fp8_gmm/utils.py:65-103).

    Slot = (group_offset + i) * stage + type with group_offset 0 for "Group1" kinds and num_groups for
    "Group2", stage 3 for forward metas and 2 for backward metas, type 1 for weights.  The
    ``kForward*`` kinds read a snapshot of the forward scale_inv taken at the end of forward, so that
    backward de-scales saved FP8 tensors with the values that produced them.
    """

    _FORWARD_OFFSET = 3
    _BACKWARD_OFFSET = 2

    def __init__(self, num_groups, fp8_meta):
        self._num_groups = num_groups
        self._fp8_meta = fp8_meta
        self._forward_scale_inv_cloned = None

    def num_groups(self):
        return self._num_groups

    def set_forward_scale_inv_cloned(self):
        self._forward_scale_inv_cloned = self._fp8_meta["scaling_fwd"].scale_inv.clone()

    _SLOT_CACHE = {}   # (tensor kind, num_groups) -> (first slot, stride): pure arithmetic, shared by all wrappers

    def _resolve(self, fp8_tensor_type, meta_tensor_type):
        kind = int(fp8_tensor_type)
        if kind >= Fp8TensorType.kForwardInputGroup1:
            assert meta_tensor_type == MetaTensorType.kScaleInv
            meta_tensor = self._forward_scale_inv_cloned
        else:
            meta = self._fp8_meta["scaling_fwd"] if kind < Fp8TensorType.kGradOutputGroup1 else self._fp8_meta["scaling_bwd"]
            if meta_tensor_type == MetaTensorType.kScale:
                meta_tensor = meta.scale
            elif meta_tensor_type == MetaTensorType.kScaleInv:
                meta_tensor = meta.scale_inv
            else:
                meta_tensor = meta.amax_history[0]
        assert meta_tensor is not None
        key = (kind, self._num_groups)
        slot = self._SLOT_CACHE.get(key)
        if slot is None:
            name = Fp8TensorType(kind).name
            group_offset = 0 if "Group1" in name else self._num_groups
            stage = self._BACKWARD_OFFSET if "GradOutput" in name else self._FORWARD_OFFSET
            type_offset = 1 if "Weight" in name else 0
            slot = self._SLOT_CACHE[key] = (group_offset * stage + type_offset, stage)
        return meta_tensor, slot[0], slot[1]

    def get_meta_tensors(self, fp8_tensor_type, meta_tensor_type):
        """List of 0-dim views, one per group (the reference's return type)."""
        t, first, stride = self._resolve(fp8_tensor_type, meta_tensor_type)
        return [t[first + i * stride] for i in range(self._num_groups)]

    def get_meta_strided(self, fp8_tensor_type, meta_tensor_type, group_start=0):
        """(1-D view starting at the slot of group ``group_start``, stride): the same slots without building G views.

        This is what the grouped C-ABI entry points consume (``base[g * stride]``).
        """
        t, first, stride = self._resolve(fp8_tensor_type, meta_tensor_type)
        return t[first + group_start * stride:], stride
