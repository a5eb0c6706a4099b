"""CUDA-graph capture / replay of a fused graph.

The same contract as xpu_graph's ``GraphRunner`` (device_graph_runner.py:11-143: static input buffers
chosen by ``init_param_callback``, refreshed by ``copy_param_callback``, one captured graph replayed by
``forward``), implemented with ``torch.cuda.CUDAGraph``. Launch-bound graphs (the encoder block and the
recsys graph issue ~10 kernels of a few microseconds each) replay without any per-op host work.

The kernels are capture-safe: the C ABI allocates nothing and never synchronises; tensor maps are encoded
on the host and passed by value as kernel parameters.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Tuple

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


class CUDAGraphRunner(torch.nn.Module):
    def __init__(self, callable_target: Callable, init_param_callback: Optional[Callable[..., List[torch.Tensor]]] = None,
                 copy_param_callback: Optional[Callable[..., bool]] = None, warmup: int = 2):
        super().__init__()
        self._callable_target = callable_target
        self._init_param_callback = init_param_callback or _default_init
        self._copy_param_callback = copy_param_callback or _default_copy
        self._warmup = warmup
        self._graph: Optional[torch.cuda.CUDAGraph] = None
        self._stream: Optional[torch.cuda.Stream] = None
        self._input_buffers: Optional[List[torch.Tensor]] = None
        self._output = None
        self._mempool = None

    @property
    def mempool(self):
        return self._mempool

    @property
    def captured(self) -> bool:
        return self._graph is not None

    def clone(self) -> "CUDAGraphRunner":
        return type(self)(self._callable_target, self._init_param_callback, self._copy_param_callback, self._warmup)

    def reset(self) -> "CUDAGraphRunner":
        self._graph, self._stream, self._input_buffers, self._output, self._mempool = None, None, None, None, None
        return self

    def capture(self, *args, memory_pool=None, clone_args: bool = False, **kwargs) -> None:
        assert self._graph is None, "Device graph has been recorded."
        if clone_args:
            args, kwargs = pytree.tree_map(lambda x: x.detach().clone() if isinstance(x, torch.Tensor) else x, (args, kwargs))
        self._input_buffers = self._init_param_callback(*args, **kwargs)
        assert self._input_buffers is not None
        self._stream = torch.cuda.Stream()
        self._mempool = memory_pool if memory_pool is not None else torch.cuda.graph_pool_handle()
        self._stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self._stream):  # warm-up outside capture: lazy initialisation must not be recorded
            for _ in range(self._warmup):
                self._callable_target(*args, **kwargs)
        torch.cuda.current_stream().wait_stream(self._stream)
        self._graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self._graph, pool=self._mempool, stream=self._stream):
            self._output = self._callable_target(*args, **kwargs)

    def forward(self, *args, **kwargs):
        assert self._graph is not None, "capture() first"
        assert self._copy_param_callback(self._input_buffers, *args, **kwargs), "inputs do not match the captured buffers"
        self._graph.replay()
        return self._output
