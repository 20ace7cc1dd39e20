"""Region timing around an unmodified Megatron ``MoELayer`` (``native/*`` regions).

The layer keeps running its own code.  A declarative list names the calls to time (attribute path on
the layer, region name, required or optional); each is shadowed on its owner *instance* by a timed
forwarder, and every shadow registers its own undo step on an ``ExitStack``, so ``remove()`` (or a
failure half-way through binding) unwinds exactly what was installed, newest first.
Reference: eplb/integration/megatron_timing.py:26-144 (same public names and regions).
"""

from __future__ import annotations

import contextlib
import functools
from typing import Callable, List, Optional, Tuple

import torch

from ..utils import profiling

# (path of the owner below the layer, method, region, required)
TIMED_CALLS: Tuple[Tuple[str, str, str, bool], ...] = (
    ("router", "forward", "native/route", True),
    ("", "dispatch", "native/dispatch", True),
    ("experts", "forward", "native/expert_gemm", True),
    ("", "combine", "native/combine", True),
    ("shared_experts", "forward", "native/shared_expert", False),
)
_MARK = "_eplb_native_timing"


def _device_of(values) -> Optional[torch.device]:
    """Device of the first tensor among the call's arguments (one level into tuples and lists)."""
    stack = list(values)
    for v in stack:
        if isinstance(v, torch.Tensor):
            return v.device
        if isinstance(v, (tuple, list)):
            for inner in v:
                if isinstance(inner, torch.Tensor):
                    return inner.device
    return None


def _shadow(undo: contextlib.ExitStack, owner, name: str, replacement: Callable) -> None:
    """Install ``replacement`` as instance attribute ``owner.name`` and register how to take it off again."""
    instance_dict = vars(owner)
    if name in instance_dict:
        previous = instance_dict[name]
        undo.callback(setattr, owner, name, previous)
    else:
        undo.callback(lambda: vars(owner).pop(name, None))
    setattr(owner, name, replacement)


class NativeMoETimingBinding:
    def __init__(self, moe_layer, *, layer_id: int, mode: str, logger: Optional[Callable[[str], None]]) -> None:
        if mode not in ("off", "observe"):
            raise ValueError("native MoE timing mode must be 'off' or 'observe'")
        if getattr(moe_layer, _MARK, None) is not None:
            raise RuntimeError("native MoE timing is already bound to this layer")
        self.moe_layer, self.layer_id, self.mode, self.logger = moe_layer, int(layer_id), mode, logger
        self.micro_batch_id = 0
        self._undo = contextlib.ExitStack()
        with contextlib.ExitStack() as guard:
            guard.push(self._undo)  # a failure below unwinds whatever was installed so far
            for path, method, region, required in TIMED_CALLS:
                owner = moe_layer if not path else getattr(moe_layer, path, None)
                target = getattr(owner, method, None) if owner is not None else None
                if not callable(target):
                    if not required:
                        continue
                    raise RuntimeError(f"cannot time {type(moe_layer).__name__}.{path + '.' if path else ''}{method}: "
                                       "no such callable on this Megatron version")
                _shadow(self._undo, owner, method, self._timed(target, region))
            _shadow(self._undo, moe_layer, "forward", self._windowed(moe_layer.forward))
            setattr(moe_layer, _MARK, self)
            self._undo.callback(lambda: vars(moe_layer).pop(_MARK, None))
            guard.pop_all()  # keep everything installed; remove() closes self._undo later

    @staticmethod
    def _timed(bound_call: Callable, region: str) -> Callable:
        @functools.wraps(bound_call)
        def forwarder(*args, **kwargs):
            with profiling.record(region, time_it=True, device=_device_of((*args, *kwargs.values()))):
                return bound_call(*args, **kwargs)

        return forwarder

    def _windowed(self, bound_forward: Callable) -> Callable:
        placeholders = {"expert_transfer": "n/a"}
        if self.mode == "off":
            placeholders.update(solver="n/a", omega_gather="n/a")

        @functools.wraps(bound_forward)
        def forwarder(*args, **kwargs):
            mb, self.micro_batch_id = self.micro_batch_id, self.micro_batch_id + 1
            profiling.begin_debug_window()
            result = bound_forward(*args, **kwargs)
            profiling.maybe_summary(self.logger, context=f"mode={self.mode} layer={self.layer_id} mb={mb}",
                                    missing=placeholders)
            return result

        return forwarder

    def remove(self) -> None:
        """Take every forwarder off again; the layer is as it was before binding."""
        self._undo.close()


def bind_native_moe_timing(model, *, mode: str, logger: Optional[Callable[[str], None]] = print
                           ) -> List[NativeMoETimingBinding]:
    layers = [m for m in model.modules() if type(m).__name__ == "MoELayer"]
    return [NativeMoETimingBinding(layer, layer_id=i, mode=mode, logger=logger) for i, layer in enumerate(layers)]
