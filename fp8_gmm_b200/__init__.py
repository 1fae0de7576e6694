"""fp8_gmm_b200: FP8 grouped GEMM for MoE training on B200 (sm_100a).

Drop-in for the Python surface of ``fp8_gmm`` (``import fp8_gmm_b200 as fp8_gmm``): the submodules
``backend``, ``grouped_linear``, ``grouped_mlp`` and ``utils`` keep the reference's names.  Importing
the package loads the C-ABI library; there is no CPU or PyTorch fallback.
"""
from . import backend, grouped_linear, grouped_mlp, utils  # noqa: F401
from .grouped_linear import GroupedLinear  # noqa: F401
from .grouped_mlp import GroupedMLP, GroupedMlp  # noqa: F401
from .recipe import DelayedScaling, Format, fp8_autocast  # noqa: F401
