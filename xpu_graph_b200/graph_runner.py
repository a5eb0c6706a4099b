"""CUDA-graph capture / replay of a fused graph: xpu_graph's ``GraphRunner`` for the ``cuda_sm100`` target.

``GraphRunner`` (device_graph_runner.py:11-143) holds the whole capture / replay contract - static input buffers
chosen by ``init_param_callback``, refreshed by ``copy_param_callback``, one captured graph replayed by ``forward`` -
and asks a backend for four things only: its graph, stream, capture-context and memory-pool types
(:33-58; NPU / MLU subclasses at :146-191). ``CUDAGraphRunner`` is that subclass for CUDA, registered under
``Target.cuda_sm100`` so that ``GraphRunner[Target.cuda_sm100]`` finds it, and under the alias ``Target.cuda`` (the
device-type spelling, which is what backends/device_graph.py:54-75 looks the runner up by).

Two additions to the inherited behaviour: default callbacks (every tensor argument gets a static buffer) and a warm-up
of the callable on a side stream before capture, so that lazy initialisation (cuBLAS handles of neighbouring aten ops,
the kernel library's one-time set-up) is not recorded into the graph.

The kernels are capture-safe: the C ABI allocates nothing and never synchronises; tensor maps are encoded on the host
and passed by value as kernel parameters.

When the xpu_graph package is not importable the same class is built on a minimal stand-in for the base class, so that
the fused graphs of this package can still be captured (bench_kernels.py, the GPU tests).
"""
from __future__ import annotations

from typing import List

import torch
import torch.utils._pytree as pytree


def _default_init(*args, **kwargs) -> List[torch.Tensor]:
    return [a for a in pytree.tree_leaves((args, kwargs)) if isinstance(a, torch.Tensor)]


def _default_copy(buffers: List[torch.Tensor], *args, **kwargs) -> bool:
    new = [a for a in pytree.tree_leaves((args, kwargs)) if isinstance(a, torch.Tensor)]
    if len(new) != len(buffers):
        return False
    for b, n in zip(buffers, new):
        if b.shape != n.shape or b.dtype != n.dtype:
            return False
        if b.data_ptr() != n.data_ptr():
            b.copy_(n, non_blocking=True)
    return True


class _CudaGraphBackend:
    """The four backend hooks of GraphRunner, plus the warm-up before capture."""

    WARMUP_CALLS = 2

    @classmethod
    def _Graph(cls, *args, **kwargs):
        return torch.cuda.CUDAGraph(*args, **kwargs)

    @classmethod
    def _Stream(cls, *args, **kwargs):
        return torch.cuda.Stream(*args, **kwargs)

    @classmethod
    def _GraphContext(cls, *args, **kwargs):
        return torch.cuda.graph(*args, **kwargs)

    @classmethod
    def _MempoolHandle(cls):
        return torch.cuda.graph_pool_handle()

    def __init__(self, callable_target, init_param_callback=None, copy_param_callback=None):
        super().__init__(callable_target, init_param_callback or _default_init, copy_param_callback or _default_copy)

    @property
    def captured(self) -> bool:
        return self._graph is not None

    def capture(self, *args, memory_pool=None, clone_args=False, **kwargs) -> None:
        assert self._graph is None, "Device graph has been recorded."
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):  # outside capture: lazy initialisation must not be recorded
            for _ in range(self.WARMUP_CALLS):
                self._callable_target(*args, **kwargs)
        torch.cuda.current_stream().wait_stream(side)
        super().capture(*args, memory_pool=memory_pool, clone_args=clone_args, **kwargs)


class _StandaloneGraphRunner(torch.nn.Module):
    """Stand-in for xpu_graph's GraphRunner where that package is absent: the part of its contract the class above
    relies on (constructor, capture, forward, clone, reset), nothing more."""

    def __init__(self, callable_target, init_param_callback=None, copy_param_callback=None):
        super().__init__()
        self._callable_target = callable_target
        self._init_param_callback = init_param_callback
        self._copy_param_callback = copy_param_callback
        self._stream = self._graph = self._input_buffers = self._output = self._mempool = None

    @property
    def mempool(self):
        return self._mempool

    def clone(self):
        return type(self)(self._callable_target, self._init_param_callback, self._copy_param_callback)

    def reset(self):
        self.__init__(self._callable_target, self._init_param_callback, self._copy_param_callback)
        return self

    def capture(self, *args, memory_pool=None, clone_args=False, **kwargs) -> None:
        assert self._graph is None, "Device graph has been recorded."
        self._stream, self._graph = self._Stream(), self._Graph()
        self._mempool = memory_pool if memory_pool else self._MempoolHandle()
        if clone_args:
            args, kwargs = pytree.tree_map(lambda x: x.detach().clone() if isinstance(x, torch.Tensor) else x, (args, kwargs))
        self._input_buffers = self._init_param_callback(*args, **kwargs)
        assert self._input_buffers is not None
        with self._GraphContext(self._graph, stream=self._stream, pool=self._mempool):
            self._output = self._callable_target(*args, **kwargs)

    def forward(self, *args, **kwargs):
        assert self._copy_param_callback(self._input_buffers, *args, **kwargs)
        self._graph.replay()
        return self._output


def _build_runner_class():
    try:
        from .target.compat import import_xpu_graph

        import_xpu_graph()
        from xpu_graph.config import Target
        from xpu_graph.device_graph_runner import GraphRunner
    except Exception:
        return type("CUDAGraphRunner", (_CudaGraphBackend, _StandaloneGraphRunner), {"__doc__": __doc__})
    from .target import TARGET_NAME, _extend_enum

    targets = [_extend_enum(Target, TARGET_NAME, TARGET_NAME), _extend_enum(Target, "cuda", "cuda")]
    registered = getattr(GraphRunner, "_registrations", {})
    if targets[0] in registered:
        return registered[targets[0]]

    class CUDAGraphRunner(_CudaGraphBackend, GraphRunner, backend=targets, anchor_class=GraphRunner):
        pass

    CUDAGraphRunner.__doc__ = __doc__
    return CUDAGraphRunner


CUDAGraphRunner = _build_runner_class()
