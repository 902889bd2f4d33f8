"""Numerical and transfer self-checks that stand in for sanitizers on shared accelerators: NaN/Inf hooks on module
outputs (cosmos_rl/utils/util.py:863-890) and the end-to-end weight-sync verifier (zero the destination, receive, and
check coverage and values: cosmos_rl/dispatcher/command.py:251-313, rollout/rollout_control.py:781-888)."""
from __future__ import annotations

from typing import Callable, Dict, List, Optional

import torch
import torch.nn as nn

from .logging import logger


class NonFiniteError(RuntimeError):
    pass


def add_nan_checks(model: nn.Module, raise_error: bool = True, on_hit: Optional[Callable[[str], None]] = None) -> List:
    """Forward hooks that look for NaN / Inf in every module's floating-point outputs and name the first module
    that produced one. Returns the hook handles (``h.remove()`` to uninstall). Costs a device sync per module: a
    debugging aid, not for production steps."""
    handles = []

    def make(name: str):
        def hook(_mod, _inp, out):
            tensors = out if isinstance(out, (tuple, list)) else (out,)
            for t in tensors:
                if torch.is_tensor(t) and t.is_floating_point() and not torch.isfinite(t).all():
                    msg = f"non-finite values in the output of {name or '<root>'} ({type(_mod).__name__})"
                    if on_hit is not None:
                        on_hit(msg)
                    if raise_error:
                        raise NonFiniteError(msg)
                    logger.error(msg)
        return hook

    for name, mod in model.named_modules():
        handles.append(mod.register_forward_hook(make(name)))
    return handles


class WeightSyncCheck:
    """Usage around one policy-to-rollout transfer::

        chk = WeightSyncCheck(flat.data)      # remembers the current weights, zeroes the destination
        ... receive ...
        report = chk.finish()                 # coverage (nothing left untouched) and equality with what was there

    ``coverage`` fails when a region of the buffer was never written (a hole in the transfer plan); ``equal`` is only
    meaningful when both sides started from the same checkpoint."""

    def __init__(self, dst: torch.Tensor, expect_equal: bool = False, slots=None):
        self.dst, self.expect_equal, self.slots = dst, expect_equal, slots
        self.before = dst.clone()
        dst.zero_()

    def finish(self, atol: float = 0.0) -> Dict[str, object]:
        got = self.dst
        holes: List[str] = []
        if self.slots:
            for s in self.slots:
                seg, ref = got[s.offset:s.offset + s.numel], self.before[s.offset:s.offset + s.numel]
                if bool((ref != 0).any()) and not bool((seg != 0).any()):
                    holes.append(s.name)
        untouched = int(((got == 0) & (self.before != 0)).sum())
        frac = untouched / max(1, got.numel())
        diff = (got.float() - self.before.float()).abs().max().item() if got.numel() else 0.0
        rep = {"untouched_fraction": frac, "holes": holes, "max_abs_diff": diff,
               "coverage_ok": not holes and frac < 1e-3, "equal": diff <= atol}
        if not rep["coverage_ok"]:
            raise RuntimeError(f"weight sync left parameters unwritten: {holes[:5] or f'{frac:.2%} of elements'}")
        if self.expect_equal and not rep["equal"]:
            raise RuntimeError(f"weight sync changed values that should be identical (max |diff| {diff:.3g})")
        logger.info("[WeightSyncCheck] coverage ok, max |new - old| = %.3g", diff)
        return rep
