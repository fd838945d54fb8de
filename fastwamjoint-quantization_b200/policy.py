"""``QuantizedPolicy``: a deployment file plus a model adapter become one object with an ``infer`` method for a
robot loop (reference: ``policy.py:13-77``).  Loading goes through ``load_deployment`` (no floating-point target
weight reaches the GPU); every ``_predict_joint_noise`` call of the model advances the denoise-call state; the
joint DiT step is replayed from CUDA graphs.  One inference at a time per instance, checked, not assumed.

The adapter is the caller's: ``build_model(model_config, device=...)`` constructs the model without weights,
``infer_kwargs(model, record, seed=...)`` turns an observation record into the arguments of
``model.infer_action``; optional ``finalize_model(model, device=...)`` and ``enable_block_fusion_dispatch(model)``.
"""
from __future__ import annotations

import logging
import threading

import torch

from .deployment import load_deployment
from .rollout_graph import LiveJointDiTGraph
from .runtime import set_wam_block_fusions
from .state import FastWAMCallTracker

_FUSABLE = ("self_attn.o", "ffn.0", "ffn.2")


class QuantizedPolicy:
    def __init__(self, deployment, adapter, *, device="cuda", construct_device="meta", cuda_graph: bool = True,
                 fuse_block: bool = False, single_graph: bool = False):
        self.model, self.state, self.metadata = load_deployment(deployment, adapter.build_model, device=device,
                                                                construct_device=construct_device)
        finalize = getattr(adapter, "finalize_model", None)
        if callable(finalize):
            finalize(self.model, device=device)
        self.adapter = adapter
        self.fused_modules = 0
        if fuse_block:
            self.fused_modules = self._enable_block_fusions()
        self.tracker = FastWAMCallTracker(self.model, self.state)
        self.tracker.install()
        self.model._wam_call_tracker = self.tracker
        if cuda_graph:
            if single_graph:
                self.state.on_device = True
            LiveJointDiTGraph(self.model, num_calls=self.state.num_calls, single_graph=single_graph).install()
        self.runtime_settings = {"construct_device": construct_device, "cuda_graph": bool(cuda_graph),
                                 "fuse_block": bool(fuse_block), "single_graph": bool(single_graph),
                                 "fused_modules": self.fused_modules}
        logging.warning("[SteerQuant runtime] %s", self.runtime_settings)
        self._busy = threading.Lock()

    def _enable_block_fusions(self) -> int:
        dispatch = getattr(self.adapter, "enable_block_fusion_dispatch", None)
        if not callable(dispatch):
            raise ValueError("Adapter must explicitly support block fusion dispatch.")
        sites = self.metadata["sites"]
        if any(site["rotation"] != "none" for site in sites):
            raise ValueError("RHT block fusion is not validated; leave fuse_block=False.")
        dispatch(self.model)
        fused = set_wam_block_fusions(self.model, True)
        expected = sum(site["operation"] in _FUSABLE for site in sites)
        if expected == 0 or fused != expected:
            raise RuntimeError("Block fusion site count does not match the deployment.")
        return fused

    def _check_request(self, kwargs: dict) -> None:
        config = self.metadata["model_config"]
        if kwargs.get("num_inference_steps") != self.state.num_calls:
            raise ValueError("infer_kwargs must explicitly match calibrated num_inference_steps.")
        if float(kwargs.get("text_cfg_scale", 1)) != 1:
            raise ValueError("Current calibration/deployment protocol requires text_cfg_scale=1.")
        if kwargs.get("sigma_shift") != config.get("sigma_shift"):
            raise ValueError("Inference sigma schedule differs from calibration configuration.")
        for key in ("action_horizon", "num_video_frames"):
            configured = config.get("model", {}).get(key)
            if configured is not None and kwargs.get(key) != configured:
                raise ValueError(f"Inference {key} differs from calibration configuration.")

    @torch.inference_mode()
    def infer(self, record, *, seed: int = 42):
        if not self._busy.acquire(blocking=False):
            raise RuntimeError("Use one policy instance per serialized inference loop.")
        try:
            self.tracker.reset()
            kwargs = self.adapter.infer_kwargs(self.model, record, seed=seed)
            self._check_request(kwargs)
            result = self.model.infer_action(**kwargs)
            if self.tracker.total_calls != self.state.num_calls:
                raise RuntimeError("Actual denoising calls differ from calibration.")
            return result
        finally:
            self.state.clear()  # also after an exception: the next call must set its own index
            self._busy.release()
