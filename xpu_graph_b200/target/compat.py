"""Makes the xpu_graph package importable and usable on recent PyTorch releases.

xpu_graph pins torch < 2.8. Three small shims, all applied from the outside (nothing in xpu_graph
is edited): an alias for a private functorch module that was renamed, a stand-in for the
``expecttest`` module its test helpers import, and a version-robust replacement of
``fx_utils.get_disable_fake_mode`` (fx_utils.py:376-386 parses ``torch.__version__[:5]``, which is
not a valid version string for two-digit minors).
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
        _DONE = True
    import xpu_graph

    return xpu_graph


def reference_available() -> bool:
    try:
        import_xpu_graph()
        return True
    except Exception:
        return False
