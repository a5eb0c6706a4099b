"""Vendor-compiler hook of the ``cuda_sm100`` target: CUDA-graph capture of the optimised graph.

xpu_graph calls ``backends/<target>.py::<target>_compile(gm, fake_inputs, is_inference=..., is_backward=...,
**vendor_compiler_config)`` when ``vendor_compiler_config`` is set (backends/__init__.py:10-29,
compiler.py:90-103). With ``{"compiler": "device_graph"}`` (the reference's name for capture/replay,
backends/device_graph.py:54-130) or ``{"mode": "cudagraphs"}`` the whole rewritten graph is captured into one
CUDA graph on its first call and replayed afterwards; parameters are used in place, the other tensor
arguments are copied into static buffers before each replay (the contract of device_graph_runner.py:112-143).
Anything else in the config returns the graph unchanged.
"""
from __future__ import annotations

import logging

import torch
import torch.utils._pytree as pytree

from ..graph_runner import CUDAGraphRunner

log = logging.getLogger("xpu_graph")


class LazyCudaGraph(torch.nn.Module):
    def __init__(self, gm: torch.nn.Module, clone_args: bool = True):
        super().__init__()
        self.gm = gm
        self.clone_args = clone_args
        self._positions = None
        self._failed = False
        self.runner = CUDAGraphRunner(gm, init_param_callback=self._init_buffers, copy_param_callback=self._copy_buffers)

    # parameters stay where they are; every other tensor argument gets a static buffer
    def _init_buffers(self, *args, **kwargs):
        flat = pytree.tree_leaves((args, kwargs))
        if self._positions is None:
            self._positions = [i for i, v in enumerate(flat)
                               if isinstance(v, torch.Tensor) and not isinstance(v, torch.nn.Parameter)]
        return [flat[i] for i in self._positions]

    def _copy_buffers(self, buffers, *args, **kwargs) -> bool:
        flat = pytree.tree_leaves((args, kwargs))
        cur = [flat[i] for i in self._positions]
        if len(cur) != len(buffers):
            return False
        for b, t in zip(buffers, cur):
            if not isinstance(t, torch.Tensor) or t.shape != b.shape or t.dtype != b.dtype:
                return False
            if t.data_ptr() != b.data_ptr():
                b.copy_(t, non_blocking=True)
        return True

    def _capture(self, *args, **kwargs):
        # clone only the non-parameter tensors, so that the captured graph reads the live parameters
        def keep_or_clone(x):
            if isinstance(x, torch.Tensor) and not isinstance(x, torch.nn.Parameter) and self.clone_args:
                return x.detach().clone()
            return x

        cargs, ckwargs = pytree.tree_map(keep_or_clone, (args, kwargs))
        self.runner.capture(*cargs, **ckwargs)

    def forward(self, *args, **kwargs):
        if self._failed:
            return self.gm(*args, **kwargs)
        if not self.runner.captured:
            try:
                self._capture(*args, **kwargs)
            except Exception as e:  # an op in the graph is not capturable: run it launch by launch
                log.warning("cuda_sm100 device_graph: capture failed (%s); running uncaptured", e)
                self._failed = True
                self.runner.reset()
                torch.cuda.synchronize()
                return self.gm(*args, **kwargs)
        out = self.runner(*args, **kwargs)
        return pytree.tree_map(lambda t: t.clone() if isinstance(t, torch.Tensor) else t, out)


def cuda_sm100_compile(gm, fake_inputs, *, is_inference: bool = False, is_backward: bool = False, **config):
    wants_graph = config.get("compiler") == "device_graph" or config.get("mode") in ("cudagraphs", "reduce-overhead")
    if not wants_graph or not is_inference:
        return gm
    on_cuda = all(t.device.type == "cuda" for t in fake_inputs if isinstance(t, torch.Tensor))
    if not on_cuda:
        return gm
    return LazyCudaGraph(gm, clone_args=bool(config.get("clone_args", True)))
