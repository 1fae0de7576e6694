"""FP8 recipe hooks: delayed scaling with an amax history, e4m3 forward / e5m2 gradients.

The reference gets these from Transformer Engine (``DelayedScaling``, ``fp8_autocast``,
``get_fp8_te_dtype`` and ``TransformerEngineBaseModule.prepare_forward`` with its ``fp8_meta``
dictionary: reference fp8_gmm/grouped_linear.py:4-5,19,124,186,206 and fp8_gmm/example.py:156-161).
Transformer Engine is not a dependency here, so this module provides the same names with the same
meaning.  The update rule is the one Transformer Engine's delayed scaling documents:

    amax      = max over the history window (``amax_compute_algo="max"``) or the latest entry
    scale     = fp8_max / amax / 2**margin     where amax is positive and finite, else unchanged
    scale_inv = 1 / scale
    history   rolled by one step with the newest slot zeroed

and runs on the GPU as one fused kernel per meta set (fp8gmm_delayed_scaling_update).  Forward metas
are refreshed at the start of a training forward from the amaxes recorded by the previous forward;
backward metas at the start of backward from the previous backward.  (The reference never triggers a
backward-side update itself; this package does, so e5m2 gradient scales follow their amaxes.)
"""
import contextlib
from dataclasses import dataclass
from enum import Enum

import torch

from . import backend
from .utils import DType


class Format(Enum):
    E4M3 = "e4m3"
    E5M2 = "e5m2"
    HYBRID = "hybrid"  # e4m3 for forward tensors, e5m2 for gradients


FP8_MAX = {torch.float8_e4m3fn: 448.0, torch.float8_e5m2: 57344.0}


@dataclass
class DelayedScaling:
    margin: int = 0
    interval: int = 1
    fp8_format: Format = Format.HYBRID
    amax_history_len: int = 1024
    amax_compute_algo: str = "max"  # "max" or "most_recent"

    def __post_init__(self):
        assert self.amax_compute_algo in ("max", "most_recent")
        assert self.amax_history_len >= 1 and self.interval >= 1


def get_fp8_te_dtype(recipe, fprop_tensor=True):
    """e4m3 for forward tensors (and for everything under Format.E4M3), e5m2 for gradients under HYBRID/E5M2."""
    if recipe.fp8_format == Format.E4M3 or (fprop_tensor and recipe.fp8_format == Format.HYBRID):
        return DType.kFloat8E4M3
    return DType.kFloat8E5M2


def get_fp8_max(recipe, fprop_tensor=True):
    return 448.0 if get_fp8_te_dtype(recipe, fprop_tensor) == DType.kFloat8E4M3 else 57344.0


_STATE = {"enabled": False, "recipe": None}


@contextlib.contextmanager
def fp8_autocast(enabled=True, fp8_recipe=None):
    """Selects the recipe the modules use inside the block (same call as Transformer Engine's)."""
    prev = dict(_STATE)
    _STATE["enabled"] = enabled
    _STATE["recipe"] = fp8_recipe if fp8_recipe is not None else DelayedScaling()
    try:
        yield
    finally:
        _STATE.update(prev)


def is_fp8_enabled():
    return _STATE["enabled"]


def get_fp8_recipe():
    return _STATE["recipe"] if _STATE["recipe"] is not None else DelayedScaling()


class Fp8Meta:
    """scale / scale_inv (n,) and amax_history (history_len, n), fp32 on the module's device."""

    def __init__(self, n, history_len, device):
        self.scale = torch.ones(n, dtype=torch.float32, device=device)
        self.scale_inv = torch.ones(n, dtype=torch.float32, device=device)
        self.amax_history = torch.zeros(history_len, n, dtype=torch.float32, device=device)


def amax_and_scale_update(fp8_meta, fwd):
    key = "scaling_fwd" if fwd else "scaling_bwd"
    meta, recipe = fp8_meta[key], fp8_meta["recipe"]
    backend.delayed_scaling_update(meta.amax_history, meta.scale, meta.scale_inv, get_fp8_max(recipe, fwd),
                                   recipe.margin, recipe.amax_compute_algo)


class Fp8GmmBaseModule(torch.nn.Module):
    """The slice of ``TransformerEngineBaseModule`` the reference modules rely on: ``fp8_meta`` and
    ``prepare_forward(inp, is_first_microbatch, num_gemms)``.  Meta vectors hold 3 slots per GEMM for
    forward (input, weight, output) and 2 per GEMM for backward, as in Transformer Engine."""

    def __init__(self):
        super().__init__()
        self.fp8_meta = {"fp8_checkpoint": False, "num_gemms": 0}
        self.fp8_meta_tensors_initialized = False

    def _init_fp8_meta(self, num_gemms, device):
        recipe = get_fp8_recipe()
        if self.fp8_meta_tensors_initialized and self.fp8_meta["num_gemms"] == num_gemms:
            if self.fp8_meta["recipe"].amax_history_len == recipe.amax_history_len:
                self.fp8_meta["recipe"] = recipe
                return
            # the window changed: keep the scales, restart the history
            for key, per in (("scaling_fwd", 3), ("scaling_bwd", 2)):
                old = self.fp8_meta[key]
                new = Fp8Meta(per * num_gemms, recipe.amax_history_len, device)
                new.scale.copy_(old.scale)
                new.scale_inv.copy_(old.scale_inv)
                self.fp8_meta[key] = new
            self.fp8_meta["recipe"] = recipe
            return
        self.fp8_meta["recipe"] = recipe
        self.fp8_meta["num_gemms"] = num_gemms
        self.fp8_meta["scaling_fwd"] = Fp8Meta(3 * num_gemms, recipe.amax_history_len, device)
        self.fp8_meta["scaling_bwd"] = Fp8Meta(2 * num_gemms, recipe.amax_history_len, device)
        self.fp8_meta["update_amax_and_scale_fwd"] = False
        self.fp8_meta["update_amax_and_scale_bwd"] = False
        self.fp8_meta["step_fwd"] = 0
        self.fp8_meta["step_bwd"] = 0
        self.fp8_meta_tensors_initialized = True

    @contextlib.contextmanager
    def prepare_forward(self, inp, is_first_microbatch, num_gemms=1):
        assert inp.is_cuda, "fp8_gmm_b200 modules run on CUDA tensors only"
        self._init_fp8_meta(num_gemms, inp.device)
        meta = self.fp8_meta
        update = is_first_microbatch is None or bool(is_first_microbatch)
        if meta["update_amax_and_scale_fwd"] and update:
            meta["step_fwd"] += 1
            if meta["step_fwd"] % meta["recipe"].interval == 0:
                amax_and_scale_update(meta, True)
        meta["update_amax_and_scale_fwd"] = self.training and torch.is_grad_enabled()
        meta["prepare_backward"] = self._prepare_backward
        yield

    def _prepare_backward(self):
        """Called by the autograd functions at the start of backward."""
        meta = self.fp8_meta
        if meta["update_amax_and_scale_bwd"]:
            meta["step_bwd"] += 1
            if meta["step_bwd"] % meta["recipe"].interval == 0:
                amax_and_scale_update(meta, False)
        meta["update_amax_and_scale_bwd"] = True

    # ---- checkpointing: FP8 state travels with state_dict so a resumed run reproduces the same bytes.
    # The extra state holds tensors, numbers and strings only, so a checkpoint written with
    # ``torch.save(model.state_dict())`` loads with ``torch.load``'s default ``weights_only=True``.
    def get_extra_state(self):
        if not self.fp8_meta_tensors_initialized:
            return None
        m = self.fp8_meta
        r = m["recipe"]
        state = {"num_gemms": m["num_gemms"],
                 "recipe": {"margin": r.margin, "interval": r.interval, "fp8_format": r.fp8_format.value,
                            "amax_history_len": r.amax_history_len, "amax_compute_algo": r.amax_compute_algo}}
        for key in ("scaling_fwd", "scaling_bwd"):
            state[key] = {"scale": m[key].scale.cpu(), "scale_inv": m[key].scale_inv.cpu(),
                          "amax_history": m[key].amax_history.cpu()}
        for key in ("update_amax_and_scale_fwd", "update_amax_and_scale_bwd", "step_fwd", "step_bwd"):
            state[key] = m[key]
        return state

    def set_extra_state(self, state):
        """Accepts what ``get_extra_state`` returns, and the key layout of Transformer Engine's modules
        (``scale_fwd`` / ``scale_inv_fwd`` / ``amax_history_fwd`` and the ``_bwd`` counterparts) when it arrives as a
        plain dictionary of tensors, so that FP8 state saved by the reference's modules can seed these."""
        if state is None:
            return
        device = next(self.parameters()).device
        m = self.fp8_meta
        if "scale_fwd" in state and "scaling_fwd" not in state:
            state = {"scaling_fwd": {"scale": state["scale_fwd"], "scale_inv": state["scale_inv_fwd"],
                                     "amax_history": state["amax_history_fwd"]},
                     "scaling_bwd": {"scale": state["scale_bwd"], "scale_inv": state["scale_inv_bwd"],
                                     "amax_history": state["amax_history_bwd"]},
                     "num_gemms": state["scale_fwd"].numel() // 3, "recipe": state.get("recipe")}
        recipe = state.get("recipe")
        if isinstance(recipe, dict):
            recipe = DelayedScaling(margin=recipe["margin"], interval=recipe["interval"], fp8_format=Format(recipe["fp8_format"]),
                                    amax_history_len=recipe["amax_history_len"], amax_compute_algo=recipe["amax_compute_algo"])
        elif recipe is None:
            recipe = DelayedScaling(amax_history_len=state["scaling_fwd"]["amax_history"].shape[0])
        m["recipe"], m["num_gemms"] = recipe, int(state["num_gemms"])
        for key, per in (("scaling_fwd", 3), ("scaling_bwd", 2)):
            meta = Fp8Meta(per * m["num_gemms"], state[key]["amax_history"].shape[0], device)
            meta.scale.copy_(state[key]["scale"])
            meta.scale_inv.copy_(state[key]["scale_inv"])
            meta.amax_history.copy_(state[key]["amax_history"])
            m[key] = meta
        defaults = {"update_amax_and_scale_fwd": True, "update_amax_and_scale_bwd": True, "step_fwd": 0, "step_bwd": 0}
        for key, default in defaults.items():
            m[key] = state.get(key, default)
        self.fp8_meta_tensors_initialized = True
