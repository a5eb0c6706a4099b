"""Makes the xpu_graph package importable and usable on recent PyTorch releases.

xpu_graph pins torch < 2.8. The shims are all applied from the outside (nothing in xpu_graph is edited): an alias
for a private functorch module that was renamed, a stand-in for the ``expecttest`` module its test helpers import,
a version-robust replacement of ``fx_utils.get_disable_fake_mode`` (fx_utils.py:376-386 parses
``torch.__version__[:5]``, which is not a valid version string for two-digit minors), and a repair of the
front-end's graph dispatch (``fx_utils.dispatch_graph``, fx_utils.py:89-261) for PyTorch releases whose AOT
functions take input / output descriptors, so that ``torch.compile(model, backend=XpuGraph(config))`` - the
reference's own entry point (compiler.py:196-237) - runs its inference path.
"""
from __future__ import annotations

import importlib
import os
import sys
import types

_DONE = False


def _find_source() -> str | None:
    env = os.environ.get("XPU_GRAPH_SRC")
    if env and os.path.isdir(os.path.join(env, "xpu_graph")):
        return env
    here = os.path.dirname(os.path.abspath(__file__))
    repo = os.path.dirname(os.path.dirname(here))
    cand = os.path.join(repo, "baseline", "_ref")  # an offline install next to this package
    return cand if os.path.isdir(os.path.join(cand, "xpu_graph")) else None


def import_xpu_graph():
    """Import xpu_graph with the shims in place. Raises ImportError if the package cannot be found."""
    global _DONE
    if not _DONE:
        import torch  # noqa: F401
        import torch._functorch._aot_autograd as aa

        old = "torch._functorch._aot_autograd.dispatch_and_compile_graph"
        if old not in sys.modules:
            try:
                importlib.import_module(old)
            except ImportError:
                sys.modules[old] = importlib.import_module("torch._functorch._aot_autograd.graph_capture")
                setattr(aa, "dispatch_and_compile_graph", sys.modules[old])
        if "expecttest" not in sys.modules:
            try:
                importlib.import_module("expecttest")
            except ImportError:
                stub = types.ModuleType("expecttest")

                class TestCase:  # minimal stand-in; only imported, never exercised
                    pass

                stub.TestCase = TestCase
                sys.modules["expecttest"] = stub
        try:
            importlib.import_module("xpu_graph")
        except ImportError:
            src = _find_source()
            if src is None:
                raise
            if src not in sys.path:
                sys.path.insert(0, src)
        import xpu_graph
        from torch._subclasses.fake_tensor import unset_fake_temporarily

        def get_disable_fake_mode():
            return unset_fake_temporarily

        from xpu_graph import fx_utils

        fx_utils.get_disable_fake_mode = get_disable_fake_mode
        for name in ("xpu_graph.passes.constant_folding", "xpu_graph.constant_manager",
                     "xpu_graph.passes.patterns.utils.submodule_manager"):
            mod = sys.modules.get(name)
            if mod is not None and hasattr(mod, "get_disable_fake_mode"):
                mod.get_disable_fake_mode = get_disable_fake_mode
        _repair_dispatch_graph(fx_utils)
        _DONE = True
    import xpu_graph

    return xpu_graph


def _repair_dispatch_graph(fx_utils) -> None:
    """Adapts the three places where fx_utils.dispatch_graph (fx_utils.py:89-261) meets a newer PyTorch.

    1. ``_collect_params_and_inputs_info`` calls ``source.name()`` (fx_utils.py:177); ``Source.name`` is a property
       now. The sources only feed guard de-duplication of duplicated inputs, so they are hidden for the duration
       of the call (the graph's ``_param_name_to_source`` and the placeholders' ``_dynamo_source``).
    2. ``run_functionalized_fw_and_collect_metadata`` wants a descriptor per flat input.
    3. ``aot_dispatch_base_graph`` wants the input descriptors too and a traced function that returns
       (outputs, output descriptors).
    Nothing is changed where the installed PyTorch still has the signatures xpu_graph was written against."""
    import inspect

    collect = fx_utils.run_functionalized_fw_and_collect_metadata
    if "flat_args_descs" not in inspect.signature(collect).parameters:
        return
    from torch._functorch._aot_autograd import descriptors as desc
    from torch._functorch._aot_autograd.utils import simple_wraps

    def collect_with_descs(f, **kwargs):
        def run(*flat_args):
            descs = [desc.PlainAOTInput(i) for i in range(len(flat_args))]
            return collect(f, flat_args_descs=descs, **kwargs)(*flat_args)

        return run

    base_graph = fx_utils.aot_dispatch_base_graph

    def base_graph_with_descs(flat_fn, flat_args, aot_config, *, fw_metadata):
        @simple_wraps(flat_fn)
        def fn_with_output_descs(*args):
            out = flat_fn(*args)
            return out, type(out)(desc.PlainAOTOutput(i) for i in range(len(out)))

        descs = [desc.PlainAOTInput(i) for i in range(len(flat_args))]
        return base_graph(fn_with_output_descs, flat_args, descs, aot_config, fw_metadata=fw_metadata)

    dispatch = fx_utils.dispatch_graph

    def dispatch_graph(gm, example_inputs, *, stage, decompositions=None):
        hidden = []
        for node in gm.graph.nodes:
            if node.op == "placeholder" and hasattr(node, "_dynamo_source"):
                hidden.append((node, node._dynamo_source))
                del node._dynamo_source
        param_sources = gm.__dict__.pop("_param_name_to_source", None)
        try:
            return dispatch(gm, example_inputs, stage=stage, decompositions=decompositions)
        finally:
            for node, source in hidden:
                node._dynamo_source = source
            if param_sources is not None:
                gm._param_name_to_source = param_sources

    fx_utils.run_functionalized_fw_and_collect_metadata = collect_with_descs
    fx_utils.aot_dispatch_base_graph = base_graph_with_descs
    fx_utils.dispatch_graph = dispatch_graph
    for name in ("xpu_graph.compiler", "xpu_graph.passes.patterns.plugin_pattern"):
        mod = sys.modules.get(name)
        if mod is not None and hasattr(mod, "dispatch_graph"):
            mod.dispatch_graph = dispatch_graph


def reference_available() -> bool:
    try:
        import_xpu_graph()
        return True
    except Exception:
        return False
