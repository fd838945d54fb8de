"""Which denoise call is running.  Same names and behaviour as the reference's ``state.py:10-71``:
modules read ``state.require()`` to pick their per-call activation scale and stream gains.

Addition: ``on_device``.  When it is set, native modules do not bake the Python index into their launches but
pass ``device_index(device)``, a one-element int32 tensor that ``set()`` keeps equal to the index; the kernels
read the schedule entry from it when they run, so one captured CUDA graph serves every call."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable

import torch


@dataclass
class DenoiseCallState:
    """Holder of the active call index in ``[0, num_calls)`` (``state.py:10-31``)."""

    num_calls: int
    index: int | None = None
    on_device: bool = False
    _mirrors: dict = field(default_factory=dict, repr=False, compare=False)

    def __post_init__(self) -> None:
        if self.num_calls <= 0:
            raise ValueError("num_calls must be positive.")

    def set(self, index: int) -> None:
        value = int(index)
        if value < 0 or value >= self.num_calls:
            raise IndexError(f"Denoise call {value} is outside [0, {self.num_calls}).")
        self.index = value
        for mirror in self._mirrors.values():
            mirror.fill_(value)  # on the current stream, ordered before the next launch or graph replay

    def device_index(self, device) -> torch.Tensor:
        """One-element int32 tensor on ``device`` holding the active index (created on first use; creating it
        allocates, so ask for it once before a stream capture)."""
        device = torch.device(device)
        mirror = self._mirrors.get(device)
        if mirror is None:
            mirror = torch.full((1,), self.require(), device=device, dtype=torch.int32)
            self._mirrors[device] = mirror
        return mirror

    def require(self) -> int:
        if self.index is None:
            raise RuntimeError("Denoise call state has not been set.")
        return self.index

    def clear(self) -> None:
        self.index = None


class FastWAMCallTracker:
    """Wraps ``model._predict_joint_noise`` so that every invocation first sets the call state to
    ``total_calls % num_calls`` (``state.py:34-71``).  Usable as a context manager."""

    HOOK = "_predict_joint_noise"

    def __init__(self, model: Any, state: DenoiseCallState) -> None:
        self.model, self.state = model, state
        self.total_calls = 0
        self._original: Callable | None = None

    def install(self) -> None:
        if self._original is not None:
            raise RuntimeError("Call tracker is already installed.")
        wrapped = getattr(self.model, self.HOOK)
        self._original = wrapped

        def tracked(*args: Any, **kwargs: Any):
            self.state.set(self.total_calls % self.state.num_calls)
            self.total_calls += 1
            return wrapped(*args, **kwargs)

        setattr(self.model, self.HOOK, tracked)

    def reset(self) -> None:
        self.total_calls = 0
        self.state.clear()

    def remove(self) -> None:
        if self._original is not None:
            setattr(self.model, self.HOOK, self._original)
            self._original = None
        self.state.clear()

    def __enter__(self) -> "FastWAMCallTracker":
        self.install()
        return self

    def __exit__(self, *_exc: object) -> None:
        self.remove()
