"""Loading a TritonLLM checkout and putting this library behind its model modules.

    from tritonllm_b200 import integration
    M = integration.load_reference("/path/to/TritonLLM")   # tritonllm.gpt_oss.triton.model
    integration.patch(M)                                    # = ops.patch(M)

``load_reference`` only imports; nothing of the checkout is copied or modified.  The reference needs
``triton`` to import (its kernels are decorated at import time) even though no Triton kernel is launched
after ``patch``.
"""
from __future__ import annotations

import importlib
import os
import sys
import types

from . import ops

_PKG = os.path.dirname(os.path.abspath(__file__))


def reference_path(path: str | None = None) -> str | None:
    """The checkout to use: the argument, else $TRITONLLM_REFERENCE, else ``baseline/_ref`` beside this
    package (an installed copy); None when none of them holds a ``tritonllm`` package."""
    for cand in (path, os.environ.get("TRITONLLM_REFERENCE"), os.path.join(os.path.dirname(_PKG), "baseline", "_ref")):
        if cand and os.path.isdir(os.path.join(cand, "tritonllm")):
            return cand
    return None


def load_reference(path: str | None = None):
    """Imports ``tritonllm`` from the checkout (which aliases its ``gpt_oss`` and ``triton_kernels``
    sub-packages as top-level modules, tritonllm/utils.py:149-159) and returns
    ``tritonllm.gpt_oss.triton.model``.  ``termcolor`` is only used for coloured prints there and is stubbed
    when it is not installed.  Raises ImportError with the reason when the checkout or one of its imports
    is missing."""
    root = reference_path(path)
    if root is None:
        raise ImportError("no TritonLLM checkout found (argument, $TRITONLLM_REFERENCE or baseline/_ref)")
    if root not in sys.path:
        sys.path.insert(0, root)
    try:
        importlib.import_module("termcolor")
    except ImportError:
        sys.modules["termcolor"] = types.ModuleType("termcolor")
    importlib.import_module("tritonllm")
    return importlib.import_module("gpt_oss.triton.model")


def patch(model_module) -> list[str]:
    """``ops.patch``: rebinds the kernel entry points the reference's model module imported."""
    return ops.patch(model_module)
