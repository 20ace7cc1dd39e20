"""Region timing around an unmodified Megatron ``MoELayer`` (``native/*`` regions).

The layer's leaf methods are wrapped, not re-implemented; ``remove()`` restores every one of them.
Reference: eplb/integration/megatron_timing.py:26-144.
"""

from __future__ import annotations

import functools
import types
from typing import Callable, List, Optional

import torch

from ..utils import profiling


def _first_device(args, kwargs):
    for v in (*args, *kwargs.values()):
        if isinstance(v, torch.Tensor):
            return v.device
        if isinstance(v, (tuple, list)):
            for item in v:
                if isinstance(item, torch.Tensor):
                    return item.device
    return None


class NativeMoETimingBinding:
    def __init__(self, moe_layer, *, layer_id: int, mode: str, logger: Optional[Callable[[str], None]]) -> None:
        if mode not in ("off", "observe"):
            raise ValueError("native MoE timing mode must be 'off' or 'observe'")
        if getattr(moe_layer, "_eplb_native_timing", None) is not None:
            raise RuntimeError("native MoE timing is already bound to this layer")
        self.moe_layer, self.layer_id, self.mode, self.logger = moe_layer, int(layer_id), mode, logger
        self.micro_batch_id = 0
        self._undo = []
        try:
            self._time(moe_layer.router, "forward", "native/route")
            self._time(moe_layer, "dispatch", "native/dispatch")
            self._time(moe_layer.experts, "forward", "native/expert_gemm")
            self._time(moe_layer, "combine", "native/combine")
            shared = getattr(moe_layer, "shared_experts", None)
            if shared is not None and callable(getattr(shared, "forward", None)):
                self._time(shared, "forward", "native/shared_expert")
            self._wrap_forward()
            moe_layer._eplb_native_timing = self
        except Exception:
            self.remove()
            raise

    def _swap(self, owner, name: str, new) -> None:
        ns = vars(owner)
        self._undo.append((owner, name, name in ns, ns.get(name)))
        setattr(owner, name, new)

    def _time(self, owner, name: str, region: str) -> None:
        original = getattr(owner, name, None)
        if not callable(original):
            who = type(owner).__name__ if owner is not None else "None"
            raise RuntimeError(f"native MoE timing requires callable {who}.{name}; "
                               "the installed Megatron MoE API is incompatible")

        @functools.wraps(original)
        def timed(_self, *args, **kwargs):
            with profiling.record(region, time_it=True, device=_first_device(args, kwargs)):
                return original(*args, **kwargs)

        self._swap(owner, name, types.MethodType(timed, owner))

    def _wrap_forward(self) -> None:
        original = self.moe_layer.forward

        @functools.wraps(original)
        def timed_forward(_self, *args, **kwargs):
            mb = self.micro_batch_id
            self.micro_batch_id += 1
            profiling.begin_debug_window()
            out = original(*args, **kwargs)
            missing = {"expert_transfer": "n/a"}
            if self.mode == "off":
                missing.update({"solver": "n/a", "omega_gather": "n/a"})
            profiling.maybe_summary(self.logger, context=f"mode={self.mode} layer={self.layer_id} mb={mb}",
                                    missing=missing)
            return out

        self._swap(self.moe_layer, "forward", types.MethodType(timed_forward, self.moe_layer))

    def remove(self) -> None:
        for owner, name, had, old in reversed(self._undo):
            if had:
                setattr(owner, name, old)
            elif name in vars(owner):
                delattr(owner, name)
        self._undo.clear()
        if getattr(self.moe_layer, "_eplb_native_timing", None) is self:
            delattr(self.moe_layer, "_eplb_native_timing")


def bind_native_moe_timing(model, *, mode: str, logger: Optional[Callable[[str], None]] = print
                           ) -> List[NativeMoETimingBinding]:
    layers = [m for m in model.modules() if type(m).__name__ == "MoELayer"]
    return [NativeMoETimingBinding(l, layer_id=i, mode=mode, logger=logger) for i, l in enumerate(layers)]
