"""Live per-denoise-call CUDA graphs around the joint DiT core.

Same contract as the reference's ``LiveJointDiTGraph`` (``rollout_graph.py:53-193``): only
``model._joint_denoise_core`` is captured, one graph per denoise-call index (the call index selects the
per-call scale and gains of every quantized linear, so it is part of what a capture records); live inputs
are copied into the captured tensors before each replay and outputs are cloned before they are returned;
a changed input layout, schedule length, guidance scale or re-entrant use is refused instead of replaying
stale data; the first replay of every graph is compared with the eager result.

``single_graph=True`` (needs the model's ``DenoiseCallState``): the state is switched to ``on_device``, so the
quantized linears read the call index from device memory; ONE graph is captured and replayed for every call
index, and its first replay at each index is compared with the eager result of that index.  ``clone_outputs=
False`` returns the captured output tensors themselves (valid until the next replay) and inputs that already
are the captured tensors (``static_inputs()``) are not copied.
"""
from __future__ import annotations

import inspect
import logging
from functools import wraps
from typing import Any

import torch

log = logging.getLogger(__name__)


def _signature(value: Any):
    """Hashable description of shapes, dtypes and constants of a call's arguments."""
    if isinstance(value, torch.Tensor):
        if value.device.type != "cuda":
            raise ValueError("Live DiT Graph inputs must be CUDA tensors.")
        return ("tensor", tuple(value.shape), value.dtype, value.device)
    if isinstance(value, dict):
        return ("dict", tuple((k, _signature(v)) for k, v in value.items()))
    if isinstance(value, (tuple, list)):
        return (type(value).__name__, tuple(_signature(v) for v in value))
    if value is None or isinstance(value, (bool, int, float, str)):
        return (type(value).__name__, value)
    raise TypeError(f"Unsupported live Graph input: {type(value).__name__}")


def _map_tensors(value, fn):
    if isinstance(value, torch.Tensor):
        return fn(value)
    if isinstance(value, dict):
        return {k: _map_tensors(v, fn) for k, v in value.items()}
    if isinstance(value, (tuple, list)):
        return type(value)(_map_tensors(v, fn) for v in value)
    return value


def _clone(value):
    return _map_tensors(value, lambda t: t.detach().clone())


def _copy(target, source) -> None:
    if isinstance(target, torch.Tensor):
        if target.data_ptr() != source.data_ptr():  # the caller may have written the captured tensor in place
            target.copy_(source)
    elif isinstance(target, dict):
        for key in target:
            _copy(target[key], source[key])
    elif isinstance(target, (tuple, list)):
        for a, b in zip(target, source):
            _copy(a, b)


class LiveJointDiTGraph:
    def __init__(self, model, *, num_calls: int = 10, warmup: int = 2, allow_numerical_mismatch: bool = False,
                 single_graph: bool = False, state=None, clone_outputs: bool = True):
        if num_calls <= 0 or warmup < 1:
            raise ValueError("Graph calls and warmup must be positive.")
        if single_graph:
            state = state if state is not None else getattr(getattr(model, "_wam_call_tracker", None), "state", None)
            if state is None:
                raise ValueError("single_graph needs the model's DenoiseCallState (state=...).")
        self.single_graph, self.state, self.clone_outputs = single_graph, state, clone_outputs
        self._validated: set[int] = set()
        self.model = model
        self.num_calls, self.warmup = num_calls, warmup
        self.allow_numerical_mismatch = allow_numerical_mismatch
        self.validation_records: list[dict] = []
        self.entries: dict[int, tuple] = {}
        self.calls = self.chunks = self.replays = 0
        self._active = self._installed = False

    # ------------------------------------------------------------------ install / remove
    def install(self):
        if self._installed or hasattr(self.model, "_rollout_graph"):
            raise RuntimeError("Live rollout Graph is already installed.")
        self.original_core = self.model._joint_denoise_core
        self.original_infer = self.model.infer_action
        self._saved = {name: self.model.__dict__.get(name) for name in ("_joint_denoise_core", "infer_action")}
        params = inspect.signature(self.original_infer)

        @wraps(self.original_infer)
        def infer(*args, **kwargs):
            bound = params.bind(*args, **kwargs)
            bound.apply_defaults()
            given = bound.arguments
            if int(given.get("num_inference_steps", self.num_calls)) != self.num_calls:
                raise ValueError("Live Graph denoising schedule changed.")
            if float(given.get("text_cfg_scale", 1.0)) != 1.0:
                raise ValueError("Live Graph currently requires text_cfg_scale=1.")
            if given.get("compile_action_infer", False):
                raise ValueError("Use live DiT Graph without compile_action_infer.")
            if self._active:
                raise RuntimeError("Concurrent/reentrant Graph inference is not supported.")
            self.calls, self._active = 0, True
            try:
                result = self.original_infer(*args, **kwargs)
                if self.calls != self.num_calls:
                    raise RuntimeError(f"Expected {self.num_calls} DiT calls, got {self.calls}.")
                self.chunks += 1
                if self.chunks == 1:
                    log.warning("[live DiT Graph] ready: %d graphs; latest inputs copied per replay; peak %.2f GiB",
                                len(self.entries), torch.cuda.max_memory_allocated() / 2**30)
                return result
            finally:
                self._active = False

        if self.single_graph:
            self._state_was_on_device = self.state.on_device
            self.state.on_device = True
        self.model._joint_denoise_core = self._call
        self.model.infer_action = infer
        self.model._rollout_graph = self
        self._installed = True
        return self

    def remove(self):
        if self._active:
            raise RuntimeError("Cannot remove Graph during inference.")
        if not self._installed:
            return
        torch.cuda.synchronize()
        for name, previous in self._saved.items():
            if previous is None:
                delattr(self.model, name)
            else:
                setattr(self.model, name, previous)
        delattr(self.model, "_rollout_graph")
        if self.single_graph:
            self.state.on_device = self._state_was_on_device
        self._validated.clear()
        self.entries.clear()
        self._installed = False

    # ------------------------------------------------------------------ the replaced core
    def static_inputs(self, index: int = 0):
        """``(args, kwargs)`` of captured input tensors of graph ``index`` (the only graph in single-graph mode):
        a caller that writes its inputs there and passes them in skips the copy-in."""
        _, static_args, static_kwargs, _, _ = self.entries[0 if self.single_graph else index]
        return static_args, static_kwargs

    def _capture(self, index: int, values, signature):
        static_args, static_kwargs = _clone(values)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(self.warmup):
                expected = self.original_core(*static_args, **static_kwargs)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()  # a pool of its own per graph: no cross-graph output lifetime
        with torch.cuda.graph(graph, stream=side):
            outputs = self.original_core(*static_args, **static_kwargs)
        graph.replay()
        torch.cuda.synchronize()
        self._validate_outputs(outputs, expected, index)
        self._validated.add(index)
        self.entries[0 if self.single_graph else index] = (signature, static_args, static_kwargs, graph, outputs)
        log.warning("[live DiT Graph] captured step %d/%d (validation mode=%s)", index + 1, self.num_calls,
                    "warn" if self.allow_numerical_mismatch else "strict")

    def _call(self, *args, **kwargs):
        if not self._active or torch.is_grad_enabled():
            raise RuntimeError("Live DiT Graph is inference-only; use model.infer_action under no_grad.")
        index = self.calls
        if index >= self.num_calls:
            raise RuntimeError("Too many joint DiT calls in this action chunk.")
        tracker = getattr(self.model, "_wam_call_tracker", None)
        if tracker is not None and tracker.state.require() != index:
            raise RuntimeError("WAM call state does not match live Graph index.")
        values = (args, kwargs)
        signature = _signature(values)
        key = 0 if self.single_graph else index
        if self.single_graph and self.state.require() != index:
            raise RuntimeError("WAM call state does not match live Graph index.")
        if key not in self.entries:
            self._capture(index, values, signature)
        captured_signature, static_args, static_kwargs, graph, outputs = self.entries[key]
        if signature != captured_signature:
            raise ValueError("Live DiT Graph input layout/constants changed; refusing stale replay.")
        _copy((static_args, static_kwargs), values)
        graph.replay()
        if self.single_graph and index not in self._validated:
            # the one graph at a call index it has not run at yet: compare with the eager result of this index
            expected = self.original_core(*static_args, **static_kwargs)
            self._validate_outputs(outputs, expected, index)
            self._validated.add(index)
        if self.allow_numerical_mismatch:  # opt-in runs still reject non-finite outputs on every replay
            for output in outputs:
                if not torch.isfinite(output).all():
                    raise RuntimeError("Nonfinite live Graph output during replay.")
        self.replays += 1
        self.calls += 1
        return _clone(outputs) if self.clone_outputs else outputs

    def _validate_outputs(self, outputs, expected, index):
        """First replay against the eager result: same count / layout, finite, close to 1e-3
        (``rollout_graph.py:157-179``).  A mismatch raises unless explicitly allowed; every check is recorded."""
        if len(outputs) != len(expected):
            raise RuntimeError("Live Graph output count changed.")
        for position, (actual, reference) in enumerate(zip(outputs, expected)):
            if actual.shape != reference.shape or actual.dtype != reference.dtype or actual.device != reference.device:
                raise RuntimeError("Live Graph output layout changed.")
            if not torch.isfinite(actual).all() or not torch.isfinite(reference).all():
                raise RuntimeError("Nonfinite live Graph output during capture validation.")
            delta = actual.float() - reference.float()
            record = {"step": index, "output": position, "max_abs": delta.abs().max().item(),
                      "rmse": delta.square().mean().sqrt().item(), "passed": True}
            try:
                torch.testing.assert_close(actual, reference, rtol=1e-3, atol=1e-3)
            except AssertionError:
                record["passed"] = False
                self.validation_records.append(record)
                if not self.allow_numerical_mismatch:
                    raise
                log.warning("[live DiT Graph] numerical mismatch ACCEPTED by explicit opt-in: %s; eager "
                            "equivalence is NOT established", record)
            else:
                self.validation_records.append(record)
