"""Loader for the reference's own code -- TEST INFRASTRUCTURE ONLY.

``load_ref_ext()`` imports the extension module that ``oracle/build_ref.py``
compiled from the reference's src/graphcuda/cpp/gcn.cpp (it exports
``gcn_conv_forward`` / ``gcn_conv_backward``, gcn.cpp:43-46).  On a machine
without the reference tree the prebuilt file in ``oracle/_ref`` is used as is.

``load_ref_python()`` additionally executes the reference's unmodified
src/graphcuda/python/gcn.py (GCNConvFunction :14-34, GCNConv :36-48) on top of
that extension, by giving its relative import ``from .. import _graphcuda`` a
synthetic parent package whose ``_graphcuda`` is the CPU-built module.  That
needs the reference tree, so it is only available where fixtures are generated.
"""
from __future__ import annotations

import importlib.machinery
import importlib.util
import os
import sys
import types

from . import build_ref

_ext = None


def ref_ext_available() -> bool:
    return os.path.exists(build_ref.built_path())


def load_ref_ext():
    global _ext
    if _ext is not None:
        return _ext
    import torch  # noqa: F401  (libtorch must be loaded before the extension)

    path = build_ref.built_path()
    if not os.path.exists(path):
        built = build_ref.build()
        if not built:
            raise ImportError("reference CPU module not built and reference tree not mounted")
    loader = importlib.machinery.ExtensionFileLoader(build_ref.NAME, path)
    spec = importlib.util.spec_from_file_location(build_ref.NAME, path, loader=loader)
    mod = importlib.util.module_from_spec(spec)
    loader.exec_module(mod)
    _ext = mod
    return mod


def load_ref_python():
    """The reference's python/gcn.py module object, bound to the CPU extension."""
    ext = load_ref_ext()
    src = os.path.join(build_ref.reference_root(), "src", "graphcuda", "python", "gcn.py")
    if not os.path.exists(src):
        raise ImportError("reference tree not mounted")
    pkg = types.ModuleType("_gc_reference")
    pkg.__path__ = []
    pkg._graphcuda = ext
    sub = types.ModuleType("_gc_reference.python")
    sub.__path__ = []
    sys.modules["_gc_reference"] = pkg
    sys.modules["_gc_reference.python"] = sub
    sys.modules["_gc_reference._graphcuda"] = ext
    spec = importlib.util.spec_from_file_location("_gc_reference.python.gcn", src)
    mod = importlib.util.module_from_spec(spec)
    mod.__package__ = "_gc_reference.python"
    sys.modules["_gc_reference.python.gcn"] = mod
    spec.loader.exec_module(mod)
    return mod
