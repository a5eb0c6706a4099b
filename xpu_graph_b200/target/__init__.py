"""The ``cuda_sm100`` vendor target of xpu_graph.

``install()`` attaches the target to an importable xpu_graph package at run time (xpu_graph itself
is not modified): it adds ``Target.cuda_sm100`` next to ``mlu`` / ``none`` / ``npu``
(config.py:11-14) and publishes the two modules that xpu_graph's target loader imports by name
(passes/patterns/targets/__init__.py:4-10 and :13-27):

    xpu_graph.passes.patterns.targets.cuda_sm100                         -> get_all_patterns(config)
    xpu_graph.passes.patterns.targets.cuda_sm100.structure_replacements  -> get_structure_replacements(config)
    xpu_graph.backends.cuda_sm100                                        -> cuda_sm100_compile (CUDA-graph capture)

``backend(config)`` returns the callable to pass to ``torch.compile(..., backend=...)``; it enters
xpu_graph through its own aot_autograd branch (compiler.py:143-153), which is the path that works on
current PyTorch releases.
"""
from __future__ import annotations

import sys
import types

from .compat import import_xpu_graph, reference_available  # noqa: F401

TARGET_NAME = "cuda_sm100"


def _extend_enum(enum_cls, name: str, value):
    if name in enum_cls.__members__:
        return enum_cls.__members__[name]
    member = object.__new__(enum_cls)
    member._name_ = name
    member._value_ = value
    enum_cls._member_map_[name] = member
    enum_cls._value2member_map_[value] = member
    enum_cls._member_names_.append(name)
    type.__setattr__(enum_cls, name, member)
    return member


def install():
    """Attach the target; returns ``Target.cuda_sm100``. Idempotent."""
    import_xpu_graph()
    from xpu_graph.config import Target

    member = _extend_enum(Target, TARGET_NAME, TARGET_NAME)
    pkg = "xpu_graph.passes.patterns.targets"
    import importlib

    importlib.import_module(pkg)
    name = f"{pkg}.{TARGET_NAME}"
    if name not in sys.modules:
        from .. import modules as _modules
        from . import patterns as _patterns

        tmod = types.ModuleType(name)
        tmod.__package__ = name
        tmod.__path__ = []  # a package, so that the sub-module import below resolves
        tmod.get_all_patterns = _patterns.get_all_patterns
        smod = types.ModuleType(f"{name}.structure_replacements")
        smod.get_structure_replacements = _modules.get_structure_replacements
        tmod.structure_replacements = smod
        sys.modules[name] = tmod
        sys.modules[f"{name}.structure_replacements"] = smod
        setattr(sys.modules[pkg], TARGET_NAME, tmod)
    bname = f"xpu_graph.backends.{TARGET_NAME}"
    if bname not in sys.modules:  # vendor-compiler hook looked up by backends/__init__.py:19-25
        import xpu_graph.backends as _backends

        from . import device_graph as _dg

        bmod = types.ModuleType(bname)
        setattr(bmod, f"{TARGET_NAME}_compile", _dg.cuda_sm100_compile)
        sys.modules[bname] = bmod
        setattr(_backends, TARGET_NAME, bmod)
    return member


def make_config(**overrides):
    """XpuGraphConfig for inference on this target (OptLevel.level2: fused kernels are not bit-exact)."""
    target = install()
    from xpu_graph.config import OptLevel, XpuGraphConfig

    kwargs = dict(is_training=False, target=target, opt_level=OptLevel.level2, enable_cache=False)
    kwargs.update(overrides)
    return XpuGraphConfig(**kwargs)


def backend(config=None, capture=None, cache=None):
    """``torch.compile`` backend: XpuGraph's inference compiler behind aot_autograd.

    ``config.enable_interceptor`` ("rtol=2e-2,atol=1e-2", the reference's syntax) wraps the compiled function in the
    reference's interceptor. ``capture``: optional dict; the optimised GraphModule is stored under ``capture['gm']``.
    ``cache``: optional XpuGraphCache (e.g. ``XpuGraphLocalCache(path)``) used when ``config.enable_cache``."""
    install()
    from torch._dynamo.backends.common import aot_autograd
    from xpu_graph import XpuGraph
    from xpu_graph.fx_utils import FxStage

    cfg = config if config is not None else make_config()
    inner = XpuGraph(cfg, cache)._get_compiler(FxStage.inference)

    def fw_compiler(gm, example_inputs):
        out = inner(gm, example_inputs)
        if capture is not None:
            capture["gm"] = out
        return out

    aot = aot_autograd(fw_compiler=fw_compiler, keep_inference_input_mutations=True)
    if getattr(cfg, "enable_interceptor", None) is None:
        return aot

    # enable_interceptor="rtol=...,atol=...": xpu_graph's own interceptor (interceptor.py:16-41, 93-179) runs the
    # Dynamo graph beside the compiled function on every call and logs / dumps divergences; its front-end attaches it
    # at compiler.py:214-225, this entry does the same around the aot_autograd result.
    def monitored_backend(dynamo_gm, example_inputs):
        import os

        from xpu_graph.interceptor import intercept

        compiled = aot(dynamo_gm, example_inputs)
        return intercept(compiled, golden_fn=dynamo_gm, fw_metadata=None, is_training=False,
                         mark=os.environ.get("RANK", "0"), config_str=cfg.enable_interceptor)

    return monitored_backend


def reference_backend(config=None, cache=None):
    """``torch.compile`` backend: the reference's own front-end, ``XpuGraph(config)`` (compiler.py:196-237), with this
    target installed - graph dispatch through ``fx_utils.dispatch_graph``, its pass manager, its runtime artifact and, if
    ``config.enable_interceptor`` is set, its interceptor with the forward metadata. On PyTorch releases newer than the
    ones xpu_graph was written against this relies on the repair in ``target/compat.py``; ``backend()`` enters the same
    inference compiler through ``aot_autograd`` instead and does not need it."""
    install()
    from xpu_graph import XpuGraph

    return XpuGraph(config if config is not None else make_config(), cache)

