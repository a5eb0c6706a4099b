"""Vendor-compiler hook of the ``cuda_sm100`` target: CUDA-graph capture of the optimised graph.

xpu_graph calls ``backends/<target>.py::<target>_compile(gm, fake_inputs, is_inference=..., is_backward=...,
**vendor_compiler_config)`` when ``vendor_compiler_config`` is set (backends/__init__.py:10-29, compiler.py:90-103).
With ``{"compiler": "device_graph"}`` (or ``{"mode": "cudagraphs" | "reduce-overhead"}``) this hook hands the graph to
the reference's own ``device_graph_compiler`` (backends/device_graph.py:54-130), as its MLU hook does
(backends/mlu.py:20-23): the graph is partitioned by capability (:14-51 - a node belongs to a partition when all its
tensors live on the device; this target's modules and ``xg_sm100`` ops qualify by that rule), every partition becomes
a lazily captured ``GraphRunner[Target.cuda]`` = ``CUDAGraphRunner``, and nodes that cannot be captured (host tensors)
stay between the partitions and run launch by launch. Parameters are used in place, the other tensor arguments are
copied into static buffers before each replay (:62-92).

Two things are added around the reference's lazy runners: a partition whose capture fails at run time (an op that
synchronises, say) falls back to launch-by-launch execution of that partition instead of failing the call, and
replayed outputs are cloned by default (``clone_outputs``; the reference returns the static output buffers, which the
next replay overwrites). Weight planes that the fp32 dense path keeps per weight (ops._weight_planes) are read as they
were at capture. Anything else in the config returns the graph unchanged.
"""
from __future__ import annotations

import logging

import torch
import torch.utils._pytree as pytree

log = logging.getLogger("xpu_graph")


class CaptureOrEager(torch.nn.Module):
    """One partition: the reference's lazy capture / replay module, with an uncaptured fallback."""

    def __init__(self, lazy: torch.nn.Module, clone_outputs: bool = True):
        super().__init__()
        self.lazy = lazy
        self.clone_outputs = clone_outputs
        self._failed = False

    @property
    def runner(self):
        return self.lazy.runner

    def forward(self, *args, **kwargs):
        eager = self.lazy.runner._callable_target
        if self._failed:
            return eager(*args, **kwargs)
        if not getattr(self.lazy, "_is_initialized", False):
            try:
                out = self.lazy(*args, **kwargs)
            except Exception as e:  # an op in the partition is not capturable: run it launch by launch
                log.warning("cuda_sm100 device_graph: capture failed (%s); this partition runs uncaptured", e)
                self._failed = True
                self.lazy.runner.reset()
                torch.cuda.synchronize()
                return eager(*args, **kwargs)
        else:
            out = self.lazy(*args, **kwargs)
        if self.clone_outputs:
            out = pytree.tree_map(lambda t: t.clone() if isinstance(t, torch.Tensor) else t, out)
        return out


def cuda_sm100_compile(gm, fake_inputs, *, is_inference: bool = False, is_backward: bool = False, **config):
    wants_graph = config.get("compiler") == "device_graph" or config.get("mode") in ("cudagraphs", "reduce-overhead")
    if not wants_graph or not is_inference:
        return gm
    on_cuda = all(t.device.type == "cuda" for t in fake_inputs if isinstance(t, torch.Tensor))
    if not on_cuda:
        return gm
    from xpu_graph.backends import device_graph

    from .. import graph_runner  # noqa: F401  (registers CUDAGraphRunner for Target.cuda_sm100 / Target.cuda)

    passed = {k: v for k, v in config.items() if k not in ("compiler", "mode", "clone_outputs")}
    fused = device_graph.device_graph_compiler(gm, fake_inputs, target="cuda", **passed)
    clone_outputs = bool(config.get("clone_outputs", True))
    for name, child in list(fused.named_children()):
        if hasattr(child, "runner") and hasattr(child, "copy_tensor_pos"):  # the reference's lazy runner modules
            setattr(fused, name, CaptureOrEager(child, clone_outputs))
    return fused
